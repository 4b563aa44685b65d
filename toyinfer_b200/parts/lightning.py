"""Linear attention with a per-head decay ("lightning" attention) and a gated output.

Per token x: q = silu(Wq x), k = silu(Wk x) [heads, dim], v = silu(Wv x) [heads, vdim].
Per head a state S [dim, vdim], zero when the sequence starts and carried from token to token
in float32: S <- decay_h S + k v^T, o = S^T q.  All heads' outputs of a token are RMS-normed
together (plain weight), multiplied by sigmoid(Wg x) and projected by Wo.

``retention`` is the same recurrence without the silu: q = Wq x, k = Wk x * dim^(-1/2), v = Wv x; each head's output
is divided by its own root mean square (no weight), all heads are multiplied by silu(Wg x) and projected by Wo (Sun et
al., "Retentive Network: A Successor to Transformer for Large Language Models", in its recurrent form with a fixed
decay per head).  Its result may be scaled and placed in the columns of a wider buffer, and its projections' rows handed
out, so that it can stand beside another mixer (parts/side_by_side.py).

The state lives in the cache's fixed-size area, one [heads, dim, vdim] float32 block per slot
(``StateRequest``): a step scans each sequence's new tokens from the state in its slot, however
many they are.  q, k, v and g come from one product.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import kernels as K
from ..kernels import lightning as KS
from ..tracing import ranged
from .base import BuildContext, Mixer, ParamSpec, StateRequest, register_part


class LightningAttention(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, dim: int, vdim: int, decay: Sequence[float],
                 eps: float, names: Optional[Dict[str, str]] = None):
        self.ctx = ctx
        self.hidden = ctx.hidden_size
        self.n_heads, self.dim, self.vdim = int(n_heads), int(dim), int(vdim)
        self.decay_values = [float(x) for x in decay]
        if len(self.decay_values) != self.n_heads:
            raise ValueError(f"lightning at {prefix!r}: {len(self.decay_values)} decays for {self.n_heads} heads")
        self.eps = float(eps)
        n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=ctx.device)
        self.w_in = self.w_o = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        H = self.n_heads
        return {
            self.names["q"]: ParamSpec((H * self.dim, self.hidden), std=0.05),
            self.names["k"]: ParamSpec((H * self.dim, self.hidden), std=0.05),
            self.names["v"]: ParamSpec((H * self.vdim, self.hidden), std=0.05),
            self.names["g"]: ParamSpec((H * self.vdim, self.hidden)),
            self.names["o"]: ParamSpec((self.hidden, H * self.vdim)),
            self.names["norm"]: ParamSpec((H * self.vdim,), role="norm", init="one_plus_normal"),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors.pop(self.names[k]) for k in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = tensors.pop(self.names["o"]).contiguous()
        self.norm_w = tensors.pop(self.names["norm"]).to(torch.float32).contiguous()

    def check_kernels(self, dtype) -> None:
        if self.dim > 128:
            raise K.KernelError(f"lightning: heads of {self.dim} query/key elements are not supported (up to 128)")

    def memory_request(self):
        return StateRequest((self.n_heads, self.dim, self.vdim), torch.float32)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("lightning",)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "state"):
            raise RuntimeError("lightning attention needs a state; the schedule gave it none")
        M = x.shape[0]
        H, qk, vd = self.n_heads, self.n_heads * self.dim, self.n_heads * self.vdim
        with ranged(batch, "mixer.qkv"):
            y = K.linear(x, self.w_in)
        q = y[:, :qk].view(M, H, self.dim)
        k = y[:, qk:2 * qk].view(M, H, self.dim)
        v = y[:, 2 * qk:2 * qk + vd].view(M, H, self.vdim)
        g = y[:, 2 * qk + vd:]
        with ranged(batch, "mixer.attention"):
            o = KS.mix(q, k, v, mem.state, self.decay, batch)
            a = KS.gated_rmsnorm(o, g, self.norm_w, self.eps)
        with ranged(batch, "mixer.out"):
            return K.linear(a, self.w_o)


class Retention(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, dim: int, vdim: int, decay: Sequence[float],
                 eps: float, names: Optional[Dict[str, str]] = None):
        self.ctx = ctx
        self.hidden = ctx.hidden_size
        self.n_heads, self.dim, self.vdim = int(n_heads), int(dim), int(vdim)
        self.decay_values = [float(x) for x in decay]
        if len(self.decay_values) != self.n_heads:
            raise ValueError(f"retention at {prefix!r}: {len(self.decay_values)} decays for {self.n_heads} heads")
        self.eps = float(eps)
        n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=ctx.device)
        self.w_in = self.w_o = None

    @property
    def n_in(self) -> int:
        return 2 * self.n_heads * (self.dim + self.vdim)

    @property
    def n_out(self) -> int:
        return self.n_heads * self.vdim

    def param_specs(self) -> Dict[str, ParamSpec]:
        H = self.n_heads
        return {
            self.names["q"]: ParamSpec((H * self.dim, self.hidden), std=0.05),
            self.names["k"]: ParamSpec((H * self.dim, self.hidden), std=0.05),
            self.names["v"]: ParamSpec((H * self.vdim, self.hidden), std=0.05),
            self.names["g"]: ParamSpec((H * self.vdim, self.hidden), std=0.05),
            self.names["o"]: ParamSpec((self.hidden, H * self.vdim), std=0.05),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors.pop(self.names[k]) for k in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = tensors.pop(self.names["o"]).contiguous()

    def check_kernels(self, dtype) -> None:
        if self.dim > 128:
            raise K.KernelError(f"retention: heads of {self.dim} query/key elements are not supported (up to 128)")

    def memory_request(self):
        return StateRequest((self.n_heads, self.dim, self.vdim), torch.float32)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("retention",)

    # -- what a mixer that stands beside another hands out (parts/side_by_side.py) --
    def in_rows(self):
        return self.w_in, None

    def out_cols(self):
        return self.w_o, None

    def mix(self, y: torch.Tensor, batch, mem, out: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
        """y [M, n_in] as projected: q, k, v and the gate's logits side by side (rows may be strided) -> the gated, normed
        heads times ``out_scale``, [M, n_out], in ``out`` when given."""
        if mem is None or not hasattr(mem, "state"):
            raise RuntimeError("retention needs a state; the schedule gave it none")
        from ..kernels import recurrent as KR
        M = y.shape[0]
        H, qk, vd = self.n_heads, self.n_heads * self.dim, self.n_heads * self.vdim
        q = y[:, :qk].view(M, H, self.dim)
        k = y[:, qk:2 * qk].view(M, H, self.dim)
        v = y[:, 2 * qk:2 * qk + vd].view(M, H, self.vdim)
        g = y[:, 2 * qk + vd:2 * qk + 2 * vd]
        o = KS.mix(q, k, v, mem.state, self.decay, batch, act="none", k_scale=float(self.dim) ** -0.5)
        return KR.head_gated_rmsnorm(o, g, None, H, self.eps, gate_act="silu", out=out, out_scale=out_scale)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        with ranged(batch, "mixer.qkv"):
            y = K.linear(x, self.w_in)
        with ranged(batch, "mixer.attention"):
            a = self.mix(y, batch, mem)
        with ranged(batch, "mixer.out"):
            return K.linear(a, self.w_o)


register_part("mixer", "lightning", LightningAttention)
register_part("mixer", "retention", Retention)
