"""The Mamba-2 mixer (state-space duality: Dao and Gu, "Transformers are SSMs").

Per token x, with inner = heads * vdim, N = state, G = groups:  [z | u | B | C | dt] = Win x  (inner, inner, G N, G N,
heads);  (u, B, C) together pass a short causal convolution per channel (``conv`` taps, a bias; the last tap weighs the
current token) and silu;  d = softplus(dt + dt_bias);  per head h (group h // (heads / G)), with S [N, vdim] zero when
the sequence starts:

    S <- exp(-exp(A_log_h) d) S + d B u_h^T;      y_h = S^T C + D_h u_h

then y * silu(z), an RMS norm over each of ``norm_groups`` equal parts of the row times a weight per channel (the gate
comes BEFORE the norm), and Wo.  Step sizes, decays, the state and the recurrence's output are float32.

What a sequence carries, one float32 row per slot (``StateRequest``): the convolution's last ``conv - 1`` inputs
[conv - 1, inner + 2 G N], then S as [heads, vdim, N].  The in-projection is one product; the convolution is the
library's short-convolution kernel with its silu; the recurrence and the gated norm are a kernel each
(kernels/recurrent.py).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import recurrent as KR
from ..tracing import ranged
from .base import BuildContext, Mixer, ParamSpec, StateRequest, register_part


class Mamba2(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, vdim: int, state: int, groups: int, conv: int,
                 norm_groups: int, eps: float, names: Optional[Dict[str, str]] = None):
        self.ctx, self.hidden = ctx, ctx.hidden_size
        self.n_heads, self.vdim, self.n_state, self.groups = int(n_heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(conv), int(norm_groups), float(eps)
        self.inner = self.n_heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state          # what the convolution runs over
        if self.groups < 1 or self.n_heads % self.groups:
            raise ValueError(f"mamba2 at {prefix!r}: {self.n_heads} heads cannot share {self.groups} groups evenly")
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2 at {prefix!r}: {self.inner} channels do not cut into {self.norm_groups} equal norm parts")
        if self.taps < 1:
            raise ValueError(f"mamba2 at {prefix!r}: a convolution of {self.taps} taps")
        n = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D", "norm": "norm",
             "o": "o"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.state_conv = 0
        self.state_s = (self.taps - 1) * self.channels
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.rate = self.skip = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        small = lambda shape, **kw: ParamSpec(shape, role="norm", **kw)
        return {
            self.names["in"]: ParamSpec((2 * self.inner + 2 * self.groups * self.n_state + self.n_heads, self.hidden), std=0.05),
            self.names["conv"]: small((self.channels, self.taps), init="normal", std=0.4),
            self.names["conv_bias"]: small((self.channels,), init="normal", std=0.1),
            self.names["dt_bias"]: small((self.n_heads,), init="normal", std=0.5, mean=-1.0),
            self.names["A_log"]: small((self.n_heads,), init="normal", std=0.5),
            self.names["D"]: small((self.n_heads,), init="one_plus_normal", std=0.2),
            self.names["norm"]: small((self.inner,), init="one_plus_normal", std=0.1),
            self.names["o"]: ParamSpec((self.hidden, self.inner), std=0.05),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda k: tensors.pop(self.names[k])
        f32 = lambda k: t(k).to(torch.float32).contiguous()
        self.w_in, self.w_o = t("in").contiguous(), t("o").contiguous()
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        self.dt_bias, self.skip, self.norm_w = f32("dt_bias"), f32("D"), f32("norm")
        self.rate = torch.exp(f32("A_log")).contiguous()

    def check_kernels(self, dtype) -> None:
        if self.n_state > 256:
            raise K.KernelError(f"mamba2: a state of {self.n_state} values per channel is not supported (up to 256)")
        if not 1 <= self.taps <= 8:
            raise K.KernelError(f"mamba2: a convolution of {self.taps} taps is not supported (1 to 8)")

    def memory_request(self):
        return StateRequest((self.state_s + self.inner * self.n_state,), torch.float32)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("mamba2",)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "state"):
            raise RuntimeError("a state-space mixer needs a state; the schedule gave it none")
        inner, ch = self.inner, self.channels
        with ranged(batch, "mixer.qkv"):
            zxbcdt = K.linear(x, self.w_in)
            xbc = KR.short_conv(zxbcdt[:, inner:inner + ch], self.conv_w, mem.state, self.state_conv, batch,
                                out_bias=self.conv_b, act="silu")
        with ranged(batch, "mixer.attention"):
            y = KR.ssd_scan(xbc, zxbcdt[:, inner + ch:], self.dt_bias, self.rate, self.skip, self.n_heads, self.groups,
                            self.n_state, self.vdim, mem.state, self.state_s, batch)
            g = KR.gate_group_rmsnorm(y, zxbcdt[:, :inner], self.norm_w, self.norm_groups, self.eps)
        with ranged(batch, "mixer.out"):
            return K.linear(g, self.w_o)


register_part("mixer", "mamba2", Mamba2)
