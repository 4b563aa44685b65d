"""Two mixers side by side on the same input:  y = left_scale * left(x) + right_scale * right(x).

Each member is a mixer of its own kind with memory of its own kind (keys and values for one, a state for the other):
the pair asks the cache with a tuple of requests and is given a tuple of views in the same order.

A member that can say which rows of an input projection it reads and which columns of an output projection it feeds
(``in_rows()``, ``out_cols()``, ``mix(y, batch, mem, out, out_scale)`` with ``n_in`` and ``n_out``; the window attention
with kept first positions and retention do) lets the pair run as ONE product in and ONE product out:

    [y_left | y_right] = [W_in,left ; W_in,right] x
    a = [left_scale * mix_left(y_left) | right_scale * mix_right(y_right)]          (each member writes its columns of a)
    y = [W_out,left | W_out,right] a + left_scale * b_left + right_scale * b_right

The scales are applied to the members' 32-bit results before they are rounded, so the sum of the two scaled outputs is
formed inside the output product's 32-bit accumulation.  Members that cannot say so run whole, one after the other, and
a kernel forms the weighted sum.

In a step of single tokens the two members' kernels are short and wait for one another for no reason: the second member
then runs on a stream of its own between the two products (an event after the input product, an event before the output
product; both are captured with the step when it is captured), so that a layer's chain is as long as the longer member's.
(In steps of many tokens the members' kernels fill the device one after the other; the same there gained nothing.)
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..tracing import ranged
from .base import BuildContext, Mixer, ParamSpec, PartSpec, build_part, register_part


class SideBySide(Mixer):
    two_streams = True          # single-token steps run the second member beside the first (tests clear it to compare)

    def __init__(self, ctx: BuildContext, prefix: str, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0, names: Optional[Dict[str, str]] = None):
        n = {"left": "left.", "right": "right."}
        n.update(names or {})
        self.hidden = ctx.hidden_size
        self.left = build_part("mixer", left, ctx, prefix + n["left"])
        self.right = build_part("mixer", right, ctx, prefix + n["right"])
        self.members = (self.left, self.right)
        self.scales = (float(left_scale), float(right_scale))
        self.joined = all(hasattr(m, "in_rows") and hasattr(m, "out_cols") and hasattr(m, "mix") for m in self.members)
        self.w_in = self.w_out = self.b_out = None
        self.pad = 0
        self._side = None           # the second member's stream, made when first needed

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for m in self.members:
            out.update(m.param_specs())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for m in self.members:
            m.bind(tensors)
        if not self.joined:
            return
        L, R = self.members
        # the left member's rows are padded to a multiple of 8 so that the right member's begin at a 16-byte boundary
        self.pad = -L.n_in % 8
        rows = [L.in_rows()[0]]
        if self.pad:
            rows.append(torch.zeros((self.pad, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        rows.append(R.in_rows()[0])
        spare = -sum(r.shape[0] for r in rows) % 8          # ... and a token's row is a whole number of 16-byte runs
        if spare:
            rows.append(torch.zeros((spare, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_out = torch.cat([L.out_cols()[0], R.out_cols()[0]], dim=1).contiguous()
        bias = None
        for m, s in zip(self.members, self.scales):
            b = m.out_cols()[1]
            if b is not None:
                bias = b.to(torch.float32) * s if bias is None else bias + b.to(torch.float32) * s
        self.b_out = bias.contiguous() if bias is not None else None

    def check_kernels(self, dtype) -> None:
        for m in self.members:
            m.check_kernels(dtype)

    @property
    def captures_start(self) -> bool:
        return all(bool(m.captures_start) for m in self.members)

    def memory_request(self):
        return tuple(m.memory_request() for m in self.members)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return tuple(m.launch_plan(n_seq, plan_len, dtype, device, n_live) for m in self.members)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if not isinstance(mem, tuple) or len(mem) != 2:
            raise RuntimeError("two mixers side by side need two memories; the schedule gave them something else")
        L, R = self.members
        if not self.joined:
            return K.weighted_sum(L.forward(x, batch, mem[0], shared), self.scales[0], R.forward(x, batch, mem[1], shared), self.scales[1])
        with ranged(batch, "mixer.qkv"):
            y = K.linear(x, self.w_in)
        M = y.shape[0]
        a = torch.empty((M, L.n_out + R.n_out), dtype=y.dtype, device=y.device)
        y_right = y[:, L.n_in + self.pad:L.n_in + self.pad + R.n_in]
        with ranged(batch, "mixer.attention"):
            if self.two_streams and batch.mode == "extend" and y.is_cuda:
                if self._side is None:
                    self._side = torch.cuda.Stream(device=y.device)
                main = torch.cuda.current_stream(y.device)
                forked, joined = torch.cuda.Event(), torch.cuda.Event()
                forked.record(main)
                self._side.wait_event(forked)
                with torch.cuda.stream(self._side):
                    R.mix(y_right, batch, mem[1], out=a[:, L.n_out:], out_scale=self.scales[1])
                    joined.record(self._side)
                L.mix(y[:, :L.n_in], batch, mem[0], out=a[:, :L.n_out], out_scale=self.scales[0])
                main.wait_event(joined)
            else:
                L.mix(y[:, :L.n_in], batch, mem[0], out=a[:, :L.n_out], out_scale=self.scales[0])
                R.mix(y_right, batch, mem[1], out=a[:, L.n_out:], out_scale=self.scales[1])
        with ranged(batch, "mixer.out"):
            return K.linear_bias(a, self.w_out, self.b_out)


register_part("mixer", "side_by_side", SideBySide)
