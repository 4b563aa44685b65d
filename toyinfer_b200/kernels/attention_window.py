"""Sliding-window attention with several score maps per head, softmax or sigmoid weights, and a logarithmic distance
term (csrc/attn_window.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import KernelError, _call, _code, _need_cuda, _ptr, _stream
from .gemm import sm_count
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float
MODES = {"softmax": 0, "sigmoid": 1}


def _pages(mem, dtype, n_kv: int, key_width: int, vdim: int, what: str):
    kp, vp, pt = mem.k_pages, mem.v_pages, mem.page_table
    if vp is None or mem.ring_rows:
        raise KernelError(f"{what}: needs keys and values of all positions (no ring, a value array)")
    if kp.dtype != dtype or vp.dtype != dtype or tuple(kp.shape[1:]) != (n_kv, mem.page_size, key_width) \
            or tuple(vp.shape[1:]) != (n_kv, mem.page_size, vdim) or not kp.is_contiguous() or not vp.is_contiguous():
        raise KernelError(f"{what}: the cache pages do not fit {n_kv} kv heads of {key_width} and {vdim} elements in {dtype}")
    return _ptr(kp), _ptr(vp), _ptr(pt), pt.shape[1], mem.page_size, kp.shape[0]


def prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
            tables, n_heads: int, n_kv: int, maps: int, dim: int, vdim: int, mem, batch) -> None:
    """qkv [M, >= heads * maps * dim + kv_heads * (maps * dim + vdim)], one projection's rows (further columns are left
    alone): adds ``bias`` (float32, q, k and v's length), norms all of q's and all of k's elements at once (weights float32
    of those lengths, or None), rotates the first ``rot`` elements of every map of q and k (``tables`` = (cos, sin, rot)
    or None), leaves the queries in place and stores keys and values in ``mem``."""
    _need_cuda(qkv, bias, q_w, k_w, what="attention_window.prepare")
    M, N = qkv.shape
    nq, nk, nv = n_heads * maps * dim, n_kv * maps * dim, n_kv * vdim
    if N < nq + nk + nv or qkv.stride(1) != 1:
        raise KernelError("attention_window.prepare: the projection's rows do not fit the heads")
    for t, n in ((bias, nq + nk + nv), (q_w, nq), (k_w, nk)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError("attention_window.prepare: biases and norm weights must be dense float32")
    cos = sin = None
    rot = max_pos = 0
    if tables is not None:
        cos, sin, rot = tables
        max_pos = cos.shape[0]
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[1] * 2 != rot or rot > dim or not cos.is_contiguous():
            raise KernelError("attention_window.prepare: rotary tables must be float32 [positions, rot / 2] with rot <= dim")
        if batch.max_pos_after > max_pos:
            raise KernelError(f"attention_window.prepare: position {batch.max_pos_after - 1} is beyond the rotary tables' {max_pos}")
    _call(_fn("ti_attn_window_prepare", [P, L, P, P, P, F, P, P, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P]),
          _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos), _ptr(sin), int(rot), int(max_pos),
          _ptr(batch.tok_pos), _ptr(batch.tok_seq), _ptr(batch.seq_slot),
          *_pages(mem, qkv.dtype, n_kv, maps * dim, vdim, "attention_window.prepare"), M, n_heads, n_kv, maps, dim, vdim,
          _code(qkv, "attention_window"), _stream())


def head_prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                 tables, pairing: str, n_heads: int, n_kv: int, dim: int, vdim: int, mem, batch) -> None:
    """As ``prepare`` for one score map and norms per head: qkv [M, >= heads * dim + kv_heads * (dim + vdim)]; adds ``bias``
    (float32, q, k and v's length), norms every head of q over its ``dim`` elements with the weight ``q_w`` (float32 [dim],
    the same for all heads; None: no norm) and every head of k with ``k_w``, rotates the first ``rot`` elements of every head
    of q and k (``tables`` = (cos, sin, rot) or None; ``pairing`` "half": element e turns with e + rot / 2, "neighbours":
    2e with 2e + 1), leaves the queries in place and stores keys and values in ``mem``."""
    _need_cuda(qkv, bias, q_w, k_w, what="attention_window.head_prepare")
    M, N = qkv.shape
    nq, nk, nv = n_heads * dim, n_kv * dim, n_kv * vdim
    if N < nq + nk + nv or qkv.stride(1) != 1:
        raise KernelError("attention_window.head_prepare: the projection's rows do not fit the heads")
    for t, n in ((bias, nq + nk + nv), (q_w, dim), (k_w, dim)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError("attention_window.head_prepare: biases and norm weights must be dense float32")
    if pairing not in ("half", "neighbours"):
        raise KernelError(f"attention_window.head_prepare: unknown pairing {pairing!r}")
    cos = sin = None
    rot = max_pos = 0
    if tables is not None:
        cos, sin, rot = tables
        max_pos = cos.shape[0]
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[1] * 2 != rot or rot > dim or not cos.is_contiguous():
            raise KernelError("attention_window.head_prepare: rotary tables must be float32 [positions, rot / 2] with rot <= dim")
        if batch.max_pos_after > max_pos:
            raise KernelError(f"attention_window.head_prepare: position {batch.max_pos_after - 1} is beyond the rotary tables' {max_pos}")
    _call(_fn("ti_attn_head_prepare", [P, L, P, P, P, F, P, P, I, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P]),
          _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos), _ptr(sin), int(rot),
          1 if pairing == "neighbours" else 0, int(max_pos), _ptr(batch.tok_pos), _ptr(batch.tok_seq), _ptr(batch.seq_slot),
          *_pages(mem, qkv.dtype, n_kv, dim, vdim, "attention_window.head_prepare"), M, n_heads, n_kv, dim, vdim,
          _code(qkv, "attention_window"), _stream())


def decode_splits(n_seq: int, n_virtual: int, per_block: int, span: int, sms: int) -> int:
    """Ranges that a single query's visible keys (``span``: the window, or the planned length when that is shorter) are
    cut into, so that the step has about four blocks per SM but no range shorter than 128 keys."""
    want = max(1, (4 * sms) // max(1, n_seq * n_virtual // per_block))
    return max(1, min(want, (span + 127) // 128, 64))


def heads_per_block(n_heads: int, n_kv: int) -> int:
    group = n_heads // n_kv
    return 4 if group % 4 == 0 else 2 if group % 2 == 0 else 1


tensor_cores = True          # tests clear this to run prompts and pieces on the CUDA-core kernel whatever their sizes


def distance_table(r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], pb: Optional[torch.Tensor], n_heads: int, window: int,
                   device) -> Optional[torch.Tensor]:
    """float32 [heads, far + 1]: what a key at distance d adds to the score under the sigmoid, pb[h] - r1[h] ln(1 + r2[h] d),
    times -log2(e) as the tensor-core kernel wants it, for every distance that a window shows (all of them share entry 0
    without a distance term).  None when a distance term meets no window: the table would have no end."""
    if r1 is not None and window <= 0:
        return None
    d = torch.arange(window if r1 is not None else 1, dtype=torch.float64, device=device)
    t = torch.zeros((n_heads, d.numel()), dtype=torch.float64, device=device)
    if r1 is not None:
        t = t - r1.double()[:, None] * torch.log1p(r2.double()[:, None] * d[None, :])
    if pb is not None:
        t = t + pb.double()[:, None]
    return (t * -1.4426950408889634).to(torch.float32).contiguous()      # the kernel works in powers of two: -log2(e) times the bias


def attend(q: torch.Tensor, maps: int, vdim: int, mem, scale: float, window: int, mode: str, batch,
           r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None, pb: Optional[torch.Tensor] = None,
           out_f32: bool = False, k: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None,
           table: Optional[torch.Tensor] = None, keep_first: int = 0, out_scale: float = 1.0,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [M, heads * maps, dim] (prepared) over the keys and values that ``mem`` holds, the step's own included ->
    [M, heads * maps * vdim] (float32 with ``out_f32``, else q's type), times ``out_scale`` before the rounding; ``out``
    (that shape, rows may be strided: columns of a wider buffer) takes the result when given.  Key j is visible to query
    i when 0 <= i - j < window, or when j <= i and j < ``keep_first`` (a sequence's first positions, which a window
    would hide, stay visible).  r1, r2: float32 [heads], the score loses r1 ln(1 + r2 (i - j)); pb: float32 [heads], added to
    the score under the sigmoid.  mode: "softmax" or "sigmoid" (weights not normalised over the keys).
    k [M, kv_heads * maps * dim], v [M, kv_heads * vdim]: the step's own keys and values as ``prepare`` left them, and
    ``table`` (``distance_table``; sigmoid mode) let prompts and pieces run on the tensor cores: bfloat16, keys and values
    of 64 or 128 elements each (csrc/attn_prefill_tc.cu); weights are then rounded to bfloat16 for the second product.
    Single tokens (a step in which every sequence goes on by one) run on the tensor-core decode kernel
    (csrc/attn_decode_mma.cu) in bfloat16 where a key row, all maps together, is as long as a value row (64 or 128), with
    the same rounding of the weights; else on the CUDA-core kernel of csrc/attn_window.cu."""
    _need_cuda(q, r1, r2, pb, what="attention_window")
    M, HV, dim = q.shape
    if HV % maps or q.stride(2) != 1 or q.stride(1) != dim:
        raise KernelError("attention_window: heads of a token must be dense")
    H = HV // maps
    for t in (r1, r2, pb):
        if t is not None and (t.dtype != torch.float32 or t.numel() != H or not t.is_contiguous()):
            raise KernelError("attention_window: per-head constants must be dense float32 [heads]")
    if mode not in MODES:
        raise KernelError(f"attention_window: unknown mode {mode!r}")
    G = mem.n_kv_heads
    pages = _pages(mem, q.dtype, G, maps * dim, vdim, "attention_window")
    code = _code(q, "attention_window")
    keep_first = int(keep_first) if window > 0 else 0
    o_dtype = torch.float32 if out_f32 else q.dtype
    if out is not None and (tuple(out.shape) != (M, HV * vdim) or out.dtype != o_dtype or out.stride(1) != 1 or not out.is_cuda):
        raise KernelError("attention_window: the result's place must be [tokens, heads * maps * vdim] of the result's type with dense rows")
    if batch.mode == "extend" and tensor_cores and q.dtype == torch.bfloat16 and maps * dim == vdim and vdim in (64, 128) \
            and dim % 8 == 0 and mem.page_size == 64 and (maps == 1 if mode == "sigmoid" else (r1 is None and pb is None)) \
            and q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0:
        # single tokens on the tensor-core kernel that the dense model decodes with (csrc/attn_decode_mma.cu): a key row as
        # long as a value row, shared by the maps; weights are rounded to bfloat16 for the second product
        from .attention import decode_splits as tile_splits
        span = min(batch.plan_len, window + keep_first + mem.page_size) if window > 0 else batch.plan_len
        splits = tile_splits(M, G, span, mem.page_size, sm_count(q.device), n_live=batch.n_real_seq)
        if out is None:
            out = torch.empty((M, HV * vdim), dtype=o_dtype, device=q.device)    # every row is a sequence's
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((M, HV, splits, vdim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((M, HV, splits, 2), dtype=torch.float32, device=q.device)
        use_table = mode == "sigmoid" and table is not None
        if use_table and (table.dtype != torch.float32 or table.dim() != 2 or table.shape[0] != H or not table.is_contiguous()):
            raise KernelError("attention_window: the distance table must be dense float32 [heads, far + 1]")
        _call(_fn("ti_attn_decode_mma_scored", [P, L, P, P, P, I, I, I, I, P, P, I, I, I, I, I, F, I, I, P, P, P, P, I, I, F, I, P, L, I, P, P, I, P]),
              _ptr(q), q.stride(0), pages[0], pages[1], pages[2], pages[3], pages[4], 0, pages[5], _ptr(batch.seq_slot),
              _ptr(batch.seq_len), M, H, G, maps, vdim, float(scale), int(window), MODES[mode], _ptr(r1), _ptr(r2), _ptr(pb),
              _ptr(table) if use_table else None, table.shape[1] - 1 if use_table else 0, keep_first, float(out_scale), splits,
              _ptr(out), out.stride(0), 1 if out_f32 else 0, _ptr(part_o), _ptr(part_ml), code, _stream())
        if splits > 1:
            _call(_fn("ti_attn_window_merge", [P, P, P, L, I, I, I, I, I, I, F, I, P]), _ptr(part_o), _ptr(part_ml), _ptr(out), out.stride(0),
                  1 if out_f32 else 0, M, HV, vdim, splits, MODES[mode], float(out_scale), code, _stream())
        return out
    if out is None:
        out = torch.zeros((M, HV * vdim), dtype=o_dtype, device=q.device)
    if batch.mode == "extend":
        span = min(batch.plan_len, window + keep_first) if window > 0 else batch.plan_len
        splits = decode_splits(M, HV, heads_per_block(H, G), span, sm_count(q.device))
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((M, HV, splits, vdim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((M, HV, splits, 2), dtype=torch.float32, device=q.device)
        _call(_fn("ti_attn_window_decode", [P, L, P, L, I, P, P, I, P, P, P, I, I, I, P, P, P, I, I, I, I, I, F, I, I, F, I, I, P, P, I, P]),
              _ptr(q), q.stride(0), _ptr(out), out.stride(0), 1 if out_f32 else 0, _ptr(batch.seq_len), _ptr(batch.seq_slot), M, *pages,
              _ptr(r1), _ptr(r2), _ptr(pb), H, G, maps, dim, vdim, float(scale), int(window), keep_first, float(out_scale), MODES[mode], splits,
              _ptr(part_o), _ptr(part_ml), code, _stream(), launches=2 if splits > 1 else 1)
        return out
    if tensor_cores and q.dtype == torch.bfloat16 and dim in (64, 128) and vdim in (64, 128) and k is not None and v is not None \
            and mem.page_size == 64 and scale > 0 and (mode == "softmax" or table is not None) and (mode == "sigmoid" or r1 is None) \
            and all(t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.stride(-1) == 1 for t in (q, k, v)) \
            and out.stride(0) % (4 if out_f32 else 8) == 0 and out.data_ptr() % 16 == 0:
        if table is not None and (table.dtype != torch.float32 or table.dim() != 2 or table.shape[0] != H or not table.is_contiguous()):
            raise KernelError("attention_window: the distance table must be dense float32 [heads, far + 1]")
        start = batch.mode == "start"
        _call(_fn("ti_attn_window_tc", [P, P, P, P, L, L, L, L, I, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P, P, I, I, I, P, I, I, F, P]),
              _ptr(q), _ptr(k), _ptr(v), _ptr(out), q.stride(0), k.stride(0), v.stride(0), out.stride(0), 1 if out_f32 else 0,
              _ptr(batch.cu_new), None if start else _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seq, batch.max_new, M, H, G,
              maps, dim, vdim, float(scale), int(window), MODES[mode], *pages, _ptr(table) if mode == "sigmoid" else None,
              table.shape[1] - 1 if (mode == "sigmoid" and table is not None) else 0, keep_first, float(out_scale), _stream())
        return out
    _call(_fn("ti_attn_window", [P, L, P, L, I, P, P, P, I, I, P, P, P, I, I, I, P, P, P, I, I, I, I, I, F, I, I, F, I, I, P]),
          _ptr(q), q.stride(0), _ptr(out), out.stride(0), 1 if out_f32 else 0, _ptr(batch.cu_new), _ptr(batch.seq_start),
          _ptr(batch.seq_slot), batch.n_seq, batch.max_new, *pages, _ptr(r1), _ptr(r2), _ptr(pb), H, G, maps, dim, vdim, float(scale),
          int(window), keep_first, float(out_scale), MODES[mode], code, _stream())
    return out


def diff_combine(a: torch.Tensor, gate: Optional[torch.Tensor], n_heads: int, vdim: int, lam: float, diff: float, eps: float,
                 out_dtype: torch.dtype) -> torch.Tensor:
    """a float32 [M, heads * 2 * vdim] (per head the two maps' outputs a1, a2), gate [M, heads] logits of ``out_dtype`` (rows
    may be strided) or None -> (a1 - lam a2) / rms(.) * (1 - diff) * sigmoid(gate), [M, heads * vdim] in ``out_dtype``."""
    _need_cuda(a, gate, what="diff_combine")
    M = a.shape[0]
    if a.dtype != torch.float32 or tuple(a.shape) != (M, n_heads * 2 * vdim) or not a.is_contiguous():
        raise KernelError("diff_combine: the maps' outputs must be dense float32 [tokens, heads * 2 * vdim]")
    if gate is not None and (tuple(gate.shape) != (M, n_heads) or gate.dtype != out_dtype or gate.stride(1) != 1):
        raise KernelError("diff_combine: the gate must be [tokens, heads] of the output's type")
    out = torch.empty((M, n_heads * vdim), dtype=out_dtype, device=a.device)
    _call(_fn("ti_diff_combine", [P, P, L, P, L, I, I, I, F, F, F, I, P]), _ptr(a), _ptr(gate), gate.stride(0) if gate is not None else 0,
          _ptr(out), out.stride(0), M, int(n_heads), int(vdim), float(lam), float(diff), float(eps),
          0 if out_dtype == torch.float32 else 1, _stream())
    return out
