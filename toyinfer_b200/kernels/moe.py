"""Mixture-of-experts feed-forward with tokens grouped by expert, and the squared-ReLU activation
(csrc/moe_grouped.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import KernelError, _call, _code, _i32, _need_cuda, _ptr, _stream
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float


def relu2(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2, elementwise."""
    _need_cuda(x, what="relu2")
    if not x.is_contiguous():
        raise KernelError("relu2: expected a dense tensor")
    out = torch.empty_like(x)
    _call(_fn("ti_relu2", [P, P, L, I, P]), _ptr(x), _ptr(out), x.numel(), _code(x, "relu2"), _stream())
    return out


def route_by_table(ids: torch.Tensor, table: torch.Tensor, n_experts: int):
    """ids int32 [M], table int32 [vocab, top] -> (perm int32 [M * top], off int32 [experts + 1]): the (token, choice)
    pairs grouped by expert."""
    _need_cuda(ids, table, what="moe_route_table")
    _i32(ids, "moe ids")
    _i32(table, "moe table")
    M = ids.numel()
    vocab, top = table.shape
    perm = torch.empty(M * top, dtype=torch.int32, device=ids.device)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=ids.device)
    scratch = torch.empty(M * top, dtype=torch.int32, device=ids.device)
    _call(_fn("ti_moe_route_table", [P, P, I, I, I, I, P, P, P, P]), _ptr(ids), _ptr(table), vocab, top, n_experts, M,
          _ptr(perm), _ptr(off), _ptr(scratch), _stream())
    return perm, off


TC_MIN_GROUP = 64          # places per expert on average from which the tcgen05 grouped product runs (groups are padded to 128)


def expert_pairs(x: torch.Tensor, perm: torch.Tensor, off: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, top: int,
                 limit: float, alpha: float, shift: float = 1.0, weight: float = 1.0):
    """Every (token, choice) pair's expert output, not yet summed: x[M, H]; w_gate_up [experts, 2 * ff, H] (an expert's gate
    rows, then its up rows); w_down [experts, H, ff]; the expert's activation is g' sigmoid(alpha g') (u' + shift) with
    g' = min(g, limit), u' = clamp(u, -limit, limit) (limit = inf, alpha = 1, shift = 0: silu(g) u).  Returns
    (z, place_of_pair): pair p's row, times ``weight``, is z[place_of_pair[p]], or z[p] when place_of_pair is None.

    bfloat16 steps with many tokens per expert pad every expert's tokens to tiles of 128 rows and run both products on
    tcgen05 (csrc/gemm_tcgen05_grouped.cu; ``weight`` is then left to the caller's sum); everything else runs the grouped
    tiles of csrc/moe_grouped.cu."""
    _need_cuda(x, perm, off, w_gate_up, w_down, what="moe")
    M, H = x.shape
    E, ff2, H2 = w_gate_up.shape
    ff = ff2 // 2
    if H2 != H or ff2 != 2 * ff or w_down.shape != (E, H, ff) or x.stride(1) != 1:
        raise KernelError("moe: the experts' matrices do not fit the tokens")
    for t in (w_gate_up, w_down):
        if t.dtype != x.dtype or not t.is_contiguous():
            raise KernelError("moe: the experts' matrices must be dense and of the tokens' dtype")
    Pn = M * top
    code = _code(x, "moe")
    if (x.dtype == torch.bfloat16 and H % 8 == 0 and ff % 8 == 0 and Pn >= TC_MIN_GROUP * E and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        rows = (Pn + 127 * E + 127) // 128 * 128
        dev = x.device
        pad_src = torch.empty(rows, dtype=torch.int32, device=dev)
        pad_of_pair = torch.empty(Pn, dtype=torch.int32, device=dev)
        tile_group = torch.empty(rows // 128, dtype=torch.int32, device=dev)
        _call(_fn("ti_moe_pad_plan", [P, P, I, I, I, I, P, P, P, P]), _ptr(perm), _ptr(off), E, Pn, top, rows, _ptr(pad_src),
              _ptr(pad_of_pair), _ptr(tile_group), _stream())
        xs = torch.empty((rows, H), dtype=x.dtype, device=dev)
        _call(_fn("ti_moe_gather_rows", [P, L, P, P, I, I, I, P]), _ptr(x), x.stride(0), _ptr(pad_src), _ptr(xs), rows, H, code, _stream())
        grouped = _fn("ti_linear_grouped_tc", [P, P, P, P, I, I, I, I, L, P])
        gu = torch.empty((rows, 2 * ff), dtype=x.dtype, device=dev)
        _call(grouped, _ptr(xs), _ptr(w_gate_up), _ptr(gu), _ptr(tile_group), rows, E, 2 * ff, H, 2 * ff, _stream())
        y = act_pair(gu, limit, alpha, shift)
        z = torch.empty((rows, H), dtype=x.dtype, device=dev)
        _call(grouped, _ptr(y), _ptr(w_down), _ptr(z), _ptr(tile_group), rows, E, H, ff, H, _stream())
        return z, pad_of_pair, True
    fn = _fn("ti_moe_grouped", [P, L, P, P, P, L, P, P, I, I, I, I, I, I, I, I, F, F, F, F, L, I, P])
    y = torch.empty((Pn, ff), dtype=x.dtype, device=x.device)
    w_up = w_gate_up[:, ff:]          # the same storage, an expert's up rows after its gate rows
    _call(fn, _ptr(x), x.stride(0), _ptr(w_gate_up), _ptr(w_up), _ptr(y), ff, _ptr(perm), _ptr(off), E, Pn, ff, H, top, 1, 0, 1,
          1.0, float(limit), float(alpha), float(shift), 2 * ff * H, code, _stream())
    z = torch.empty((Pn, H), dtype=x.dtype, device=x.device)
    _call(fn, _ptr(y), ff, _ptr(w_down), None, _ptr(z), H, _ptr(perm), _ptr(off), E, Pn, H, ff, top, 0, 1, 0,
          float(weight), 0.0, 0.0, 0.0, 0, code, _stream())
    return z, None, False


def act_pair(gu: torch.Tensor, limit: float, alpha: float, shift: float = 1.0) -> torch.Tensor:
    """gu [rows, 2 * ff] dense, a row's gate values and then its up values -> g' sigmoid(alpha g') (u' + shift) with
    g' = min(g, limit), u' = clamp(u, -limit, limit), [rows, ff], in 32-bit with one rounding."""
    _need_cuda(gu, what="moe_act_pair")
    if gu.dim() != 2 or gu.shape[1] % 2 or not gu.is_contiguous():
        raise KernelError("moe_act_pair: expected a dense [rows, 2 * ff] tensor")
    rows, ff = gu.shape[0], gu.shape[1] // 2
    y = torch.empty((rows, ff), dtype=gu.dtype, device=gu.device)
    _call(_fn("ti_moe_act_pair", [P, P, L, I, F, F, F, I, P]), _ptr(gu), _ptr(y), rows, ff, float(limit), float(alpha), float(shift),
          _code(gu, "moe"), _stream())
    return y


def experts_ffn(x: torch.Tensor, perm: torch.Tensor, off: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, top: int,
                limit: float, alpha: float, weight: float) -> torch.Tensor:
    """``expert_pairs`` with shift 1, every pair's output times ``weight``, summed per token in the order of its choices
    -> [M, H]."""
    M, H = x.shape
    z, place, padded = expert_pairs(x, perm, off, w_gate_up, w_down, top, limit, alpha, 1.0, weight)
    code = _code(x, "moe")
    if padded:
        out = torch.empty((M, H), dtype=x.dtype, device=x.device)
        _call(_fn("ti_moe_combine_indexed", [P, P, P, I, I, I, F, I, P]), _ptr(z), _ptr(place), _ptr(out), M, H, top, float(weight),
              code, _stream())
        return out
    if top == 1:
        return z
    out = torch.empty((M, H), dtype=x.dtype, device=x.device)
    _call(_fn("ti_moe_combine", [P, P, I, I, I, I, P]), _ptr(z), _ptr(out), M, H, top, code, _stream())
    return out


def route_softmax(z: torch.Tensor, correction, n_experts: int, top: int, n_groups: int = 0, keep: int = 0, scale: float = 1.0):
    """z float32 [M, >= experts] (rows may be strided) -> (perm int32 [M * top], off int32 [experts + 1], weight float32
    [M * top]): with s = softmax(z) over the experts, every token's ``top`` experts by s + correction (float32 [experts] or
    None), chosen only among the ``keep`` best of ``n_groups`` equal runs of neighbouring experts (a run's score: its
    largest s + correction; ``n_groups`` <= 1: no runs); a pair's weight is its s over the sum of the token's chosen s, times
    ``scale``.  The pairs come out grouped by expert (csrc/moe_router.cu)."""
    _need_cuda(z, correction, what="moe_route_softmax")
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1 or z.shape[1] < n_experts:
        raise KernelError("moe_route_softmax: the router's logits must be float32 [tokens, experts] with dense rows")
    if correction is not None and (correction.dtype != torch.float32 or tuple(correction.shape) != (n_experts,) or not correction.is_contiguous()):
        raise KernelError("moe_route_softmax: the correction must be dense float32 [experts]")
    M = z.shape[0]
    dev = z.device
    perm = torch.empty(M * top, dtype=torch.int32, device=dev)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(M * top, dtype=torch.int32, device=dev)
    weight = torch.empty(M * top, dtype=torch.float32, device=dev)
    _call(_fn("ti_moe_route_softmax", [P, L, P, I, I, I, I, F, I, P, P, P, P, P]), _ptr(z), z.stride(0), _ptr(correction), int(n_experts),
          int(top), int(n_groups), int(keep), float(scale), M, _ptr(perm), _ptr(off), _ptr(scratch), _ptr(weight), _stream())
    return perm, off, weight


def route_topk(z: torch.Tensor, n_experts: int, top: int):
    """z float32 [M, >= experts] (rows may be strided; the first ``n_experts`` columns are the router's logits) ->
    (perm int32 [M * top], off int32 [experts + 1], score float32 [M * top], score squared): every token's ``top``
    experts by sigmoid(z), the (token, choice) pairs grouped by expert (csrc/moe_router.cu)."""
    _need_cuda(z, what="moe_route_topk")
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1 or z.shape[1] < n_experts:
        raise KernelError("moe_route_topk: the router's logits must be float32 [tokens, experts] with dense rows")
    M = z.shape[0]
    dev = z.device
    perm = torch.empty(M * top, dtype=torch.int32, device=dev)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(M * top, dtype=torch.int32, device=dev)
    score = torch.empty(M * top, dtype=torch.float32, device=dev)
    score2 = torch.empty(M * top, dtype=torch.float32, device=dev)
    _call(_fn("ti_moe_route_topk", [P, L, I, I, I, P, P, P, P, P, P]), _ptr(z), z.stride(0), int(n_experts), int(top), M, _ptr(perm),
          _ptr(off), _ptr(scratch), _ptr(score), _ptr(score2), _stream())
    return perm, off, score, score2


def experts_relu2(x: torch.Tensor, perm: torch.Tensor, off: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, top: int):
    """Every pair's Wdown relu(Wup x)^2 with its expert's matrices: x [M, H]; w_up [experts, ff, H]; w_down [experts, H, ff].
    Returns (z, place_of_pair): pair p's row is z[place_of_pair[p]], or z[p] when place_of_pair is None.  The same two
    ways as ``experts_ffn``: padded groups on tcgen05 for many tokens per expert, the grouped tiles otherwise."""
    _need_cuda(x, perm, off, w_up, w_down, what="moe")
    M, H = x.shape
    E, ff, H2 = w_up.shape
    if H2 != H or w_down.shape != (E, H, ff) or x.stride(1) != 1:
        raise KernelError("moe: the experts' matrices do not fit the tokens")
    for t in (w_up, w_down):
        if t.dtype != x.dtype or not t.is_contiguous():
            raise KernelError("moe: the experts' matrices must be dense and of the tokens' dtype")
    Pn = M * top
    code = _code(x, "moe")
    dev = x.device
    if (x.dtype == torch.bfloat16 and H % 8 == 0 and ff % 8 == 0 and Pn >= TC_MIN_GROUP * E and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        rows = (Pn + 127 * E + 127) // 128 * 128
        pad_src = torch.empty(rows, dtype=torch.int32, device=dev)
        pad_of_pair = torch.empty(Pn, dtype=torch.int32, device=dev)
        tile_group = torch.empty(rows // 128, dtype=torch.int32, device=dev)
        _call(_fn("ti_moe_pad_plan", [P, P, I, I, I, I, P, P, P, P]), _ptr(perm), _ptr(off), E, Pn, top, rows, _ptr(pad_src),
              _ptr(pad_of_pair), _ptr(tile_group), _stream())
        xs = torch.empty((rows, H), dtype=x.dtype, device=dev)
        _call(_fn("ti_moe_gather_rows", [P, L, P, P, I, I, I, P]), _ptr(x), x.stride(0), _ptr(pad_src), _ptr(xs), rows, H, code, _stream())
        grouped = _fn("ti_linear_grouped_tc", [P, P, P, P, I, I, I, I, L, P])
        u = torch.empty((rows, ff), dtype=x.dtype, device=dev)
        _call(grouped, _ptr(xs), _ptr(w_up), _ptr(u), _ptr(tile_group), rows, E, ff, H, ff, _stream())
        y = relu2(u)
        z = torch.empty((rows, H), dtype=x.dtype, device=dev)
        _call(grouped, _ptr(y), _ptr(w_down), _ptr(z), _ptr(tile_group), rows, E, H, ff, H, _stream())
        return z, pad_of_pair
    fn = _fn("ti_moe_grouped", [P, L, P, P, P, L, P, P, I, I, I, I, I, I, I, I, F, F, F, F, L, I, P])
    u = torch.empty((Pn, ff), dtype=x.dtype, device=dev)
    _call(fn, _ptr(x), x.stride(0), _ptr(w_up), None, _ptr(u), ff, _ptr(perm), _ptr(off), E, Pn, ff, H, top, 1, 0, 0,
          1.0, 0.0, 0.0, 0.0, 0, code, _stream())
    y = relu2(u)
    z = torch.empty((Pn, H), dtype=x.dtype, device=dev)
    _call(fn, _ptr(y), ff, _ptr(w_down), None, _ptr(z), H, _ptr(perm), _ptr(off), E, Pn, H, ff, top, 0, 1, 0,
          1.0, 0.0, 0.0, 0.0, 0, code, _stream())
    return z, None


def combine_gated(z: torch.Tensor, place_of_pair, pair_w, shared_out, gate_logit, M: int, top: int) -> torch.Tensor:
    """out[m] = sum_j pair_w[m * top + j] * z[place of that pair] + sigmoid(gate_logit[m]) * shared_out[m].  z [places, H];
    pair_w float32 [M * top] or None; shared_out [M, H] or None; gate_logit float32 [M] (may be strided) or None."""
    _need_cuda(z, place_of_pair, pair_w, shared_out, gate_logit, what="moe_combine_gated")
    H = z.shape[1]
    if not z.is_contiguous() or (shared_out is not None and (tuple(shared_out.shape) != (M, H) or shared_out.dtype != z.dtype
                                                             or not shared_out.is_contiguous())):
        raise KernelError("moe_combine_gated: the outputs must be dense and of one type")
    if gate_logit is not None and (gate_logit.dtype != torch.float32 or gate_logit.dim() != 1 or gate_logit.shape[0] != M):
        raise KernelError("moe_combine_gated: the gate's logits must be float32 [tokens]")
    out = torch.empty((M, H), dtype=z.dtype, device=z.device)
    _call(_fn("ti_moe_combine_gated", [P, P, P, P, P, L, P, I, I, I, I, P]), _ptr(z), _ptr(place_of_pair), _ptr(pair_w), _ptr(shared_out),
          _ptr(gate_logit), gate_logit.stride(0) if gate_logit is not None else 0, _ptr(out), M, H, int(top), _code(z, "moe"), _stream())
    return out
