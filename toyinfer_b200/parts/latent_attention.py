"""Multi-head latent attention with a sliding window and per-head sinks.

Per token x: q = Wq x, head by head [``dim`` plain | ``rot_dim`` rotated]; d = Wdkv x;
c = rms(d[:kv_rank]) * w (the latent), r = rotate(d[kv_rank:]) (one rotated key part for all
heads).  Head h's key is [Wuk_h c | r], its value Wuv_h c, the score (q_h . k_h) * scale with
``scale`` as given.  A position sees itself and the ``window - 1`` before it (0: all); the
softmax's denominator also holds exp(sink_h).  Output Wo on the heads' values side by side.

The cache keeps [c | r] per position, one row for all heads (a request without values: the
value is read out of the same row).  The kernels never form keys or values per head: the
query is carried through Wuk into the latent space, the attention runs over the cached rows,
and the result goes through Wuv (kernels/latent.py).  q and d come from one product.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import latent as KL
from ..tracing import ranged
from .base import BuildContext, KVRequest, Mixer, ParamSpec, register_part


class LatentAttention(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, eps: float, position: Optional[str] = None, window: int = 0, sinks: bool = True,
                 names: Optional[Dict[str, str]] = None):
        self.ctx = ctx
        self.hidden = ctx.hidden_size
        self.n_heads, self.dim, self.rot, self.vdim, self.rank = int(n_heads), int(dim), int(rot_dim), int(vdim), int(kv_rank)
        if min(self.n_heads, self.vdim, self.rank) <= 0 or self.dim < 0 or self.rot < 0 or self.dim + self.rot <= 0:
            raise ValueError(f"latent attention at {prefix!r}: sizes must be positive")
        if self.rot % 2:
            raise ValueError(f"latent attention at {prefix!r}: the rotated part must be even, got {self.rot}")
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window or 0)
        self.sinks = bool(sinks)
        n = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink", "o": "o"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.pos = None
        if self.rot:
            try:
                self.pos = ctx.positions[position]
                if getattr(self.pos, "pairing", "half") != "half":
                    raise ValueError(f"attention at {prefix!r}: its kernels turn elements (e, e + rot / 2) together, the position encoding {position!r} pairs neighbours")
            except KeyError:
                raise ValueError(f"latent attention at {prefix!r} names unknown position encoding {position!r}") from None
            tables = getattr(self.pos, "dim", None)
            if tables is not None and tables != self.rot:
                raise ValueError(f"latent attention at {prefix!r}: the position encoding rotates {tables} elements, not {self.rot}")
        self.w_qd = self.w_uk = self.w_uv = self.w_o = self.norm_w = self.sink = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, hd, W = self.n_heads, self.dim + self.rot, self.rank + self.rot
        s = {
            self.names["q"]: ParamSpec((H * hd, self.hidden)),
            self.names["dkv"]: ParamSpec((W, self.hidden)),
            self.names["dkv_norm"]: ParamSpec((self.rank,), role="norm", init="one_plus_normal"),
            self.names["uk"]: ParamSpec((H * self.dim, self.rank), std=0.1),
            self.names["uv"]: ParamSpec((H * self.vdim, self.rank), std=0.1),
            self.names["o"]: ParamSpec((self.hidden, H * self.vdim)),
        }
        if self.sinks:
            s[self.names["sink"]] = ParamSpec((H,), role="norm", init="normal", std=1.0)
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_qd = torch.cat([tensors.pop(self.names["q"]), tensors.pop(self.names["dkv"])], dim=0).contiguous()
        self.w_uk = tensors.pop(self.names["uk"]).contiguous()
        self.w_uv = tensors.pop(self.names["uv"]).contiguous()
        self.w_o = tensors.pop(self.names["o"]).contiguous()
        # for steps of whole prompts on the tensor cores: both up-projections as one matrix, and the output projection
        # with columns of zeros where a head of D elements holds nothing
        self.w_ukv = self.w_o_padded = None
        D = KL.prompt_heads(self.dim, self.rot, self.vdim)
        if self.w_o.dtype == torch.bfloat16 and D:
            self.w_ukv = torch.cat([self.w_uk, self.w_uv], dim=0).contiguous()
            if D == self.vdim:
                self.w_o_padded = self.w_o
            else:
                wide = torch.zeros((self.hidden, self.n_heads, D), dtype=self.w_o.dtype, device=self.w_o.device)
                wide[:, :, : self.vdim] = self.w_o.view(self.hidden, self.n_heads, self.vdim)
                self.w_o_padded = wide.view(self.hidden, self.n_heads * D).contiguous()
        self.norm_w = tensors.pop(self.names["dkv_norm"]).to(torch.float32).contiguous()
        self.sink = tensors.pop(self.names["sink"]).to(torch.float32).contiguous() if self.sinks else None

    def check_kernels(self, dtype) -> None:
        if self.rank > 1024:
            raise K.KernelError(f"latent_attention: a latent of {self.rank} elements is not supported (up to 1,024)")
        smem = (64 * (self.rank + self.rot + 1) + 32 * 33) * 4
        if smem > 227 * 1024:
            raise K.KernelError(f"latent_attention: rows of {self.rank + self.rot} elements need {smem} bytes of shared memory")

    def memory_request(self):
        return KVRequest(1, self.rank + self.rot, self.window, values=False)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("latent", KL.plan(n_seq, self.n_heads, self.window, plan_len, device))    # the split of a sequence's keys over blocks

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "k_pages"):
            raise RuntimeError("latent attention needs its cache rows; the schedule gave it none")
        M = x.shape[0]
        H, hd = self.n_heads, self.dim + self.rot
        with ranged(batch, "mixer.qkv"):
            qd = K.linear(x, self.w_qd)
        q = qd[:, : H * hd].view(M, H, hd)
        d = qd[:, H * hd:]
        with ranged(batch, "mixer.attention"):
            tables = self.pos.rotary_tables() if self.pos is not None else None
            D = 0
            if KL.single_eligible(q, self.rank, self.rot, batch, mem):
                # one token each: three launches from the projection's output to the output projection's input
                a = KL.attention_single(d, q, self.rank, self.rot, self.norm_w, self.eps, tables, self.w_uk, self.w_uv, self.vdim,
                                        self.scale, self.window, self.sink, batch, mem)
            else:
                # In a ring, a long run of new rows overwrites positions that the run's first queries still read:
                # such a step stores after its attention (which takes the step's own rows from the step anyway).
                store_first = not (batch.mode == "mixed" and mem.ring_rows > 0)
                lat = KL.prep(d, q, self.rank, self.rot, self.norm_w, self.eps, tables, batch, mem if store_first else None)
                D = KL.prompt_eligible(q, lat, self.rank, self.rot, self.vdim, batch) if self.w_ukv is not None else 0
                if D:
                    a = KL.attention_prompt(q, lat, self.w_ukv, self.vdim, self.rank, self.rot, self.scale, self.window,
                                            self.sink, batch, D)
                else:
                    a = KL.attention(q, lat, self.w_uk, self.w_uv, self.vdim, self.rank, self.rot, self.scale, self.window,
                                     self.sink, batch, mem)
                if not store_first:
                    KL.store(lat, batch, mem)
        with ranged(batch, "mixer.out"):
            return K.linear(a, self.w_o_padded if D else self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
