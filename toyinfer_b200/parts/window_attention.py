"""Three sliding-window attention mixers over keys and values of different sizes, on shared kernels
(kernels/attention_window.py): attention with sigmoid weights, differential attention, and softmax attention under a
window that keeps a sequence's first positions visible.

Both: q = Wq x [heads, maps, dim], k = Wk x [kv_heads, maps, dim], v = Wv x [kv_heads, vdim]; query head h reads kv head
h // (heads / kv_heads); key j is visible to the query at i when 0 <= i - j < window (window 0: every j <= i); y = Wo o.

``sigmoid_attention`` (one map): the projections have biases; ALL of q's elements are normed at once, and all of k's
(x * rsqrt(mean(x^2) + eps) * w, a weight per element); no rotation;

    s_ij = (q_i . k_j) * scale - r1_h ln(1 + r2_h (i - j));      w_ij = sigmoid(s_ij + pb_h);      o_i = sum_j w_ij v_j

with no normalisation over the keys.  The distance term and the biases are each optional.

``diff_attention`` (two maps; Ye et al., "Differential Transformer"): the first ``rot_dim`` elements of every map of q
and k are rotated by the token's position (a position encoding of the model, by name); each map is a softmax attention
of its own over the same values, a1 and a2; with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (one number per layer),

    o = a1 - lambda a2;      o <- o / sqrt(mean(o^2) + eps) * (1 - diff);      o <- o * sigmoid(Wg x)_h

per head.  The gate's rows ride with the q, k, v projection.

``kept_window_attention`` (one map): biases on all four projections (each optional); every head of q and of k normed over
its own elements with one weight [dim] for all heads; the first ``rot_dim`` elements of every head of q and k rotated by
the token's position, in the pairing that the position encoding names; key j is visible to the query at i when
0 <= i - j < window, or when j <= i and j < keep_first: the first ``keep_first`` positions of a sequence stay visible to
every later query, at their own positions; softmax over the visible keys.  Its result may be scaled and placed in the
columns of a wider buffer, and its projections' rows handed out, so that it can stand beside another mixer
(parts/side_by_side.py).

Keys and values of all positions live in the cache; a step first stores its own, then attends over the pages,
whatever mix of new and cached tokens it brings.  Only the last ``window`` positions are ever read.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import attention_window as KW
from ..kernels.gemm import sm_count
from ..tracing import ranged
from .base import BuildContext, KVRequest, Mixer, ParamSpec, register_part


class _WindowAttention(Mixer):
    captures_start = True
    maps = 1
    mode = "softmax"

    def _sizes(self, ctx, prefix, n_heads, n_kv_heads, dim, vdim, scale, window, eps):
        if n_kv_heads < 1 or n_heads % n_kv_heads:
            raise ValueError(f"attention at {prefix!r}: {n_heads} heads cannot share {n_kv_heads} kv heads evenly")
        if int(window) < 0:
            raise ValueError(f"attention at {prefix!r}: a window of {window} positions (0: every earlier position)")
        self.ctx, self.hidden, self.prefix = ctx, ctx.hidden_size, prefix
        self.n_heads, self.n_kv, self.dim, self.vdim = int(n_heads), int(n_kv_heads), int(dim), int(vdim)
        self.scale, self.window, self.eps = float(scale), int(window), float(eps)

    def check_kernels(self, dtype) -> None:
        if max(self.dim, self.vdim) > 256:
            raise K.KernelError(f"attention: heads of {self.dim} and {self.vdim} elements are not supported (up to 256)")

    def memory_request(self):
        # every position is kept (pages, no ring); the window bounds what is read
        return KVRequest(self.n_kv, self.maps * self.dim, 0, True, self.vdim if self.vdim != self.maps * self.dim else 0)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        span = min(plan_len, self.window) if self.window > 0 else plan_len
        return ("window", KW.decode_splits(n_seq, self.n_heads * self.maps, KW.heads_per_block(self.n_heads, self.n_kv), span,
                                           sm_count(device)))

    def _memory(self, mem):
        if mem is None or not hasattr(mem, "k_pages"):
            raise RuntimeError("attention needs key/value memory; the schedule gave it none")


class SigmoidAttention(_WindowAttention):
    mode = "sigmoid"

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 window: int, eps: float, biases: bool = True, row_norm: bool = True, distance: bool = True, head_bias: bool = True,
                 names: Optional[Dict[str, str]] = None):
        self._sizes(ctx, prefix, n_heads, n_kv_heads, dim, vdim, scale, window, eps)
        self.biases, self.row_norm, self.distance, self.head_bias = bool(biases), bool(row_norm), bool(distance), bool(head_bias)
        n = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "r1": "r1", "r2": "r2", "pb": "pb",
             "bias": ".b"}
        n.update(names or {})
        self.n = n
        self.w_qkv = self.w_o = self.b_qkv = self.q_w = self.k_w = self.r1 = self.r2 = self.pb = self.table = None

    def _name(self, k: str, bias: bool = False) -> str:
        return self.prefix + self.n[k] + (self.n["bias"] if bias else "")

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        small = lambda shape, **kw: ParamSpec(shape, role="norm", **kw)
        s = {self._name("q"): ParamSpec((H * d, self.hidden), std=0.05), self._name("k"): ParamSpec((G * d, self.hidden), std=0.05),
             self._name("v"): ParamSpec((G * vd, self.hidden), std=0.05), self._name("o"): ParamSpec((self.hidden, H * vd), std=0.05)}
        if self.biases:
            for k, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
                s[self._name(k, True)] = small((rows,), init="normal", std=0.1)
        if self.row_norm:
            s[self._name("q_norm")] = small((H * d,), init="one_plus_normal", std=0.1)
            s[self._name("k_norm")] = small((G * d,), init="one_plus_normal", std=0.1)
        if self.distance:
            s[self._name("r1")] = small((H,), init="normal", std=0.2, mean=0.5)
            s[self._name("r2")] = small((H,), init="normal", std=0.05, mean=0.5)
        if self.head_bias:
            s[self._name("pb")] = small((H,), init="normal", std=0.5, mean=-2.0)
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda name: tensors.pop(name)
        f32 = lambda name: t(name).to(torch.float32).contiguous()
        self.w_qkv = torch.cat([t(self._name(k)) for k in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = t(self._name("o")).contiguous()
        if self.biases:
            self.b_qkv = torch.cat([f32(self._name(k, True)) for k in ("q", "k", "v")]).contiguous()
        if self.row_norm:
            self.q_w, self.k_w = f32(self._name("q_norm")), f32(self._name("k_norm"))
        if self.distance:
            self.r1, self.r2 = f32(self._name("r1")), f32(self._name("r2"))
        if self.head_bias:
            self.pb = f32(self._name("pb"))
        # what a distance adds under the sigmoid, for the tensor-core kernel: a row per head as long as the window
        self.table = KW.distance_table(self.r1, self.r2, self.pb, self.n_heads, self.window, self.w_o.device)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        self._memory(mem)
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        with ranged(batch, "mixer.qkv"):
            qkv = K.linear(x, self.w_qkv)
        M = qkv.shape[0]
        with ranged(batch, "mixer.attention"):
            KW.prepare(qkv, self.b_qkv, self.q_w, self.k_w, self.eps, None, H, G, 1, d, vd, mem, batch)
            a = KW.attend(qkv[:, :H * d].view(M, H, d), 1, vd, mem, self.scale, self.window, "sigmoid", batch,
                          r1=self.r1, r2=self.r2, pb=self.pb, k=qkv[:, H * d:(H + G) * d], v=qkv[:, (H + G) * d:(H + G) * d + G * vd],
                          table=self.table)
        with ranged(batch, "mixer.out"):
            return K.linear(a, self.w_o)


class DiffAttention(_WindowAttention):
    maps = 2

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 window: int, eps: float, diff: float, position: Optional[str] = None, gate: bool = True,
                 names: Optional[Dict[str, str]] = None):
        self._sizes(ctx, prefix, n_heads, n_kv_heads, dim, vdim, scale, window, eps)
        self.diff, self.gate = float(diff), bool(gate)
        self.position = None
        if position is not None:
            if position not in ctx.positions:
                raise ValueError(f"attention at {prefix!r} names position encoding {position!r}, which the model does not have")
            self.position = ctx.positions[position]
            if getattr(self.position, "pairing", "half") != "half":
                raise ValueError(f"attention at {prefix!r}: its kernel turns elements (e, e + rot / 2) together, the position encoding {position!r} pairs neighbours")
        n = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.w_in = self.w_o = None
        self.lam = 0.0

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        s = {self.names["q"]: ParamSpec((H * 2 * d, self.hidden), std=0.05), self.names["k"]: ParamSpec((G * 2 * d, self.hidden), std=0.05),
             self.names["v"]: ParamSpec((G * vd, self.hidden), std=0.05), self.names["o"]: ParamSpec((self.hidden, H * vd), std=0.05)}
        for k in ("lq1", "lk1", "lq2", "lk2"):
            s[self.names[k]] = ParamSpec((d,), role="norm", init="normal", std=0.1)
        if self.gate:
            s[self.names["g"]] = ParamSpec((H, self.hidden), std=0.05)
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda k: tensors.pop(self.names[k])
        f64 = lambda k: t(k).to(torch.float64)
        # q, k, v and the gate's rows as one matrix: one product per token row
        # (rows of zeros bring the product's rows to a multiple of 16 bytes, which the tensor-core kernel's loads need)
        parts = [t(k) for k in (("q", "k", "v", "g") if self.gate else ("q", "k", "v"))]
        spare = -sum(p.shape[0] for p in parts) % 8
        if spare:
            parts.append(torch.zeros((spare, self.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = t("o").contiguous()
        self.lam = math.exp(float((f64("lq1") * f64("lk1")).sum())) - math.exp(float((f64("lq2") * f64("lk2")).sum())) + self.diff

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        self._memory(mem)
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        with ranged(batch, "mixer.qkv"):
            qkvg = K.linear(x, self.w_in)
        M = qkvg.shape[0]
        nq, nkv = H * 2 * d, G * (2 * d + vd)
        with ranged(batch, "mixer.attention"):
            tables = self.position.rotary_tables() if self.position is not None else None
            KW.prepare(qkvg, None, None, None, self.eps, tables, H, G, 2, d, vd, mem, batch)
            a = KW.attend(qkvg[:, :nq].view(M, 2 * H, d), 2, vd, mem, self.scale, self.window, "softmax", batch, out_f32=True,
                          k=qkvg[:, nq:nq + G * 2 * d], v=qkvg[:, nq + G * 2 * d:nq + nkv])
            o = KW.diff_combine(a, qkvg[:, nq + nkv:nq + nkv + H] if self.gate else None, H, vd, self.lam, self.diff, self.eps, qkvg.dtype)
        with ranged(batch, "mixer.out"):
            return K.linear(o, self.w_o)


class KeptWindowAttention(_WindowAttention):
    """Softmax attention under a sliding window that keeps the first ``keep_first`` positions visible (see the module's text)."""

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 window: int, eps: float, keep_first: int = 0, position: Optional[str] = None, biases: bool = True,
                 head_norm: bool = True, names: Optional[Dict[str, str]] = None):
        self._sizes(ctx, prefix, n_heads, n_kv_heads, dim, vdim, scale, window, eps)
        if int(keep_first) < 0:
            raise ValueError(f"attention at {prefix!r}: {keep_first} kept first positions")
        self.keep_first = int(keep_first) if self.window > 0 else 0
        self.biases, self.head_norm = bool(biases), bool(head_norm)
        self.position = None
        if position is not None:
            if position not in ctx.positions:
                raise ValueError(f"attention at {prefix!r} names position encoding {position!r}, which the model does not have")
            self.position = ctx.positions[position]
        n = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "bias": ".b"}
        n.update(names or {})
        self.n = n
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.q_w = self.k_w = None

    def _name(self, k: str, bias: bool = False) -> str:
        return self.prefix + self.n[k] + (self.n["bias"] if bias else "")

    @property
    def n_in(self) -> int:
        return self.n_heads * self.dim + self.n_kv * (self.dim + self.vdim)

    @property
    def n_out(self) -> int:
        return self.n_heads * self.vdim

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        small = lambda shape, **kw: ParamSpec(shape, role="norm", **kw)
        s = {self._name("q"): ParamSpec((H * d, self.hidden), std=0.05), self._name("k"): ParamSpec((G * d, self.hidden), std=0.05),
             self._name("v"): ParamSpec((G * vd, self.hidden), std=0.05), self._name("o"): ParamSpec((self.hidden, H * vd), std=0.05)}
        if self.biases:
            for k, rows in (("q", H * d), ("k", G * d), ("v", G * vd), ("o", self.hidden)):
                s[self._name(k, True)] = small((rows,), init="normal", std=0.1)
        if self.head_norm:
            s[self._name("q_norm")] = small((d,), init="one_plus_normal", std=0.1)
            s[self._name("k_norm")] = small((d,), init="one_plus_normal", std=0.1)
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda name: tensors.pop(name)
        f32 = lambda name: t(name).to(torch.float32).contiguous()
        self.w_qkv = torch.cat([t(self._name(k)) for k in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = t(self._name("o")).contiguous()
        if self.biases:
            self.b_qkv = torch.cat([f32(self._name(k, True)) for k in ("q", "k", "v")]).contiguous()
            self.b_o = f32(self._name("o", True))
        if self.head_norm:
            self.q_w, self.k_w = f32(self._name("q_norm")), f32(self._name("k_norm"))

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        span = min(plan_len, self.window + self.keep_first) if self.window > 0 else plan_len
        return ("kept_window", KW.decode_splits(n_seq, self.n_heads, KW.heads_per_block(self.n_heads, self.n_kv), span, sm_count(device)))

    # -- what a mixer that stands beside another hands out (parts/side_by_side.py) --
    def in_rows(self):
        """(the rows of the projection that ``mix`` reads, float32 biases of those rows or None)."""
        return self.w_qkv, self.b_qkv

    def out_cols(self):
        """(the output projection [hidden, n_out], its float32 bias or None)."""
        return self.w_o, self.b_o

    def mix(self, qkv: torch.Tensor, batch, mem, out: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
        """qkv [M, n_in] as projected, without biases (rows may be strided; changed in place) -> the heads' outputs times
        ``out_scale``, [M, n_out], in ``out`` when given."""
        self._memory(mem)
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        M = qkv.shape[0]
        tables = self.position.rotary_tables() if self.position is not None else None
        pairing = getattr(self.position, "pairing", "half")
        KW.head_prepare(qkv, self.b_qkv, self.q_w, self.k_w, self.eps, tables, pairing, H, G, d, vd, mem, batch)
        return KW.attend(qkv[:, :H * d].view(M, H, d), 1, vd, mem,
                         self.scale, self.window, "softmax", batch, k=qkv[:, H * d:(H + G) * d],
                         v=qkv[:, (H + G) * d:(H + G) * d + G * vd], keep_first=self.keep_first, out_scale=out_scale, out=out)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        with ranged(batch, "mixer.qkv"):
            qkv = K.linear(x, self.w_qkv)
        with ranged(batch, "mixer.attention"):
            a = self.mix(qkv, batch, mem)
        with ranged(batch, "mixer.out"):
            return K.linear_bias(a, self.w_o, self.b_o)


register_part("mixer", "sigmoid_attention", SigmoidAttention)
register_part("mixer", "kept_window_attention", KeptWindowAttention)
register_part("mixer", "diff_attention", DiffAttention)
