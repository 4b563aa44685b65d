"""Recurrent mixers' kernels: the short convolution with its state (csrc/short_conv.cu), the real-gated linear
recurrent unit (csrc/rglru.cu), the gated delta rule and the per-head gated norm (csrc/delta_rule.cu).

Every state lives in one float32 tensor per schedule entry, [slots, n]: a kernel is given the address of its part of
slot 0 and the distance between slots."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import KernelError, _call, _code, _need_cuda, _ptr, _stream
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float
ACTS = {None: 0, "none": 0, "silu": 1}


def _state_part(state: torch.Tensor, offset: int, size: int, what: str):
    """(address of slot 0's part, floats between slots) of ``state`` [slots, n] float32."""
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or offset < 0 or offset + size > state.shape[1]:
        raise KernelError(f"{what}: the state must be dense float32 [slots, n] with room for {size} values at {offset}")
    return state.data_ptr() + 4 * offset, state.shape[1]


def _vec(t: Optional[torch.Tensor], n: int, what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
        raise KernelError(f"{what} must be dense float32 of {n} values")


def short_conv(x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, state_offset: int, batch,
               in_bias: Optional[torch.Tensor] = None, out_bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """x [M, C] (rows may be strided) -> act(causal convolution per channel + out_bias) [M, C]; the inputs are x + in_bias,
    and the last taps - 1 of them per sequence live in ``state`` [slots, n] from ``state_offset`` on."""
    _need_cuda(x, taps, state, in_bias, out_bias, what="short_conv")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("short_conv: rows must be dense")
    M, C = x.shape
    if taps.dtype != torch.float32 or taps.dim() != 2 or taps.shape[0] != C or not taps.is_contiguous():
        raise KernelError(f"short_conv: the filters must be dense float32 [{C}, taps]")
    n = taps.shape[1]
    _vec(in_bias, C, "short_conv: the input bias")
    _vec(out_bias, C, "short_conv: the output bias")
    if act not in ACTS:
        raise KernelError(f"short_conv: unknown activation {act!r}")
    base, stride = _state_part(state, state_offset, (n - 1) * C, "short_conv")
    out = torch.zeros((M, C), dtype=x.dtype, device=x.device)       # rows that are nobody's stay zero
    _call(_fn("ti_short_conv", [P, L, P, P, P, I, P, L, P, L, P, P, I, I, I, I, I, P]),
          _ptr(x), x.stride(0), _ptr(in_bias), _ptr(taps), _ptr(out_bias), ACTS[act], base, stride, _ptr(out), C,
          _ptr(batch.cu_new), _ptr(batch.seq_slot), batch.n_seq, batch.max_new, C, n, _code(x, "short_conv"), _stream(),
          launches=2 if (batch.max_new > 64 and n > 1) else 1)
    return out


RGLRU_CHUNKED_FROM = 256        # new tokens of one sequence from which a step runs the chunked form (three launches)


def rglru_scan(gates: torch.Tensor, u: torch.Tensor, z: torch.Tensor, gate_bias_r: torch.Tensor, gate_bias_i: torch.Tensor,
               z_bias: Optional[torch.Tensor], rate: torch.Tensor, block: int, state: torch.Tensor, state_offset: int, batch) -> torch.Tensor:
    """gates float32 [M, 2 C] (per gate block of ``block`` channels: its recurrence-gate logits, then its input-gate
    logits), u [M, C] the convolved input, z [M, C] the other branch before its bias and gelu -> S_t * gelu(z_t) [M, C]."""
    _need_cuda(gates, u, z, gate_bias_r, gate_bias_i, z_bias, rate, state, what="rglru_scan")
    M, C = u.shape
    if gates.dtype != torch.float32 or tuple(gates.shape) != (M, 2 * C) or not gates.is_contiguous():
        raise KernelError(f"rglru_scan: the gate logits must be dense float32 [{M}, {2 * C}]")
    if z.shape != u.shape or z.dtype != u.dtype or u.stride(1) != 1 or z.stride(1) != 1 or C % block:
        raise KernelError("rglru_scan: the two branches do not fit together")
    for t, what in ((gate_bias_r, "recurrence-gate bias"), (gate_bias_i, "input-gate bias"), (z_bias, "branch bias"), (rate, "rate")):
        _vec(t, C, f"rglru_scan: the {what}")
    base, stride = _state_part(state, state_offset, C, "rglru_scan")
    out = torch.zeros((M, C), dtype=u.dtype, device=u.device)
    if batch.max_new >= RGLRU_CHUNKED_FROM:
        chunks = (batch.max_new + 127) // 128
        scratch = torch.empty((batch.n_seq, chunks, 2, C), dtype=torch.float32, device=u.device)
        _call(_fn("ti_rglru_scan_chunked", [P, P, L, P, L, P, P, P, P, P, L, P, P, P, P, I, I, I, I, I, P]),
              _ptr(gates), _ptr(u), u.stride(0), _ptr(z), z.stride(0), _ptr(gate_bias_r), _ptr(gate_bias_i), _ptr(z_bias), _ptr(rate),
              base, stride, _ptr(out), _ptr(scratch), _ptr(batch.cu_new), _ptr(batch.seq_slot), batch.n_seq, batch.max_new, C, int(block),
              _code(u, "rglru_scan"), _stream(), launches=3)
        return out
    _call(_fn("ti_rglru_scan", [P, P, L, P, L, P, P, P, P, P, L, P, P, P, I, I, I, I, P]),
          _ptr(gates), _ptr(u), u.stride(0), _ptr(z), z.stride(0), _ptr(gate_bias_r), _ptr(gate_bias_i), _ptr(z_bias), _ptr(rate),
          base, stride, _ptr(out), _ptr(batch.cu_new), _ptr(batch.seq_slot), batch.n_seq, C, int(block), _code(u, "rglru_scan"), _stream())
    return out


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_logit: torch.Tensor, dt_bias: torch.Tensor,
               rate: torch.Tensor, beta_logit: torch.Tensor, state: torch.Tensor, state_offset: int, batch) -> torch.Tensor:
    """q, k [M, qk_heads, dim] and v [M, heads, vdim] after their convolutions (not yet unit vectors); decay_logit float32
    [M, heads * dim]; dt_bias float32 [heads * dim]; rate float32 [heads]; beta_logit [M, heads].  Returns float32
    [M, heads * vdim]; the state [heads, dim, vdim] per slot is left as it is after the step's tokens."""
    _need_cuda(q, k, v, decay_logit, dt_bias, rate, beta_logit, state, what="delta_rule")
    M, G, dim = q.shape
    H, vdim = v.shape[1], v.shape[2]
    if k.shape != q.shape or v.shape[0] != M or k.dtype != q.dtype or v.dtype != q.dtype or H % G:
        raise KernelError("delta_rule: q, k and v do not fit together")
    for t in (q, k, v):
        if t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise KernelError("delta_rule: heads of a token must be dense")
    if decay_logit.dtype != torch.float32 or tuple(decay_logit.shape) != (M, H * dim) or not decay_logit.is_contiguous():
        raise KernelError(f"delta_rule: the decay logits must be dense float32 [{M}, {H * dim}]")
    if tuple(beta_logit.shape) != (M, H) or beta_logit.dtype != q.dtype or beta_logit.stride(1) != 1:
        raise KernelError("delta_rule: the write-strength logits must be [tokens, heads] of the tokens' type")
    _vec(dt_bias, H * dim, "delta_rule: the decay bias")
    _vec(rate, H, "delta_rule: the rates")
    base, stride = _state_part(state, state_offset, H * dim * vdim, "delta_rule")
    o = torch.zeros((M, H * vdim), dtype=torch.float32, device=q.device)
    # unit queries and keys, decays and betas of all tokens, made by a kernel of their own before the recurrence
    scratch = torch.empty(M * (2 * G * dim + H * dim + H), dtype=torch.float32, device=q.device)
    _call(_fn("ti_delta_rule_scan", [P, P, P, L, L, L, P, P, P, P, L, P, P, L, P, P, P, I, I, I, I, I, I, I, P]),
          _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(decay_logit), _ptr(dt_bias), _ptr(rate),
          _ptr(beta_logit), beta_logit.stride(0), _ptr(o), base, stride, _ptr(scratch), _ptr(batch.cu_new), _ptr(batch.seq_slot),
          batch.n_seq, M, H, G, dim, vdim, _code(q, "delta_rule"), _stream(), launches=2)
    return o


def head_gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, w: Optional[torch.Tensor], n_heads: int, eps: float,
                       gate_act: str = "sigmoid", out: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
    """o float32 [M, heads * vdim], gate [M, heads * vdim] logits of the engine's type (rows may be strided), w float32
    [vdim] or None (ones) -> o / rms(o) per head * w * act(gate) * out_scale, in the gate's type; ``gate_act`` is "sigmoid"
    or "silu".  ``out`` [M, heads * vdim] (rows may be strided, e.g. columns of a wider buffer) takes the result."""
    _need_cuda(o, gate, w, out, what="head_gated_rmsnorm")
    M, N = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or tuple(gate.shape) != (M, N) or gate.stride(1) != 1 or N % n_heads:
        raise KernelError("head_gated_rmsnorm: o must be dense float32 and the gate of its shape")
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError(f"head_gated_rmsnorm: unknown gate function {gate_act!r}")
    if w is not None:
        _vec(w, N // n_heads, "head_gated_rmsnorm: the weight")
    if out is None:
        out = torch.empty((M, N), dtype=gate.dtype, device=o.device)
    elif tuple(out.shape) != (M, N) or out.dtype != gate.dtype or out.stride(1) != 1:
        raise KernelError("head_gated_rmsnorm: the result's place must be [tokens, heads * vdim] of the gate's type with dense rows")
    _call(_fn("ti_head_gated_rmsnorm", [P, P, L, P, P, L, I, I, I, F, I, F, I, P]), _ptr(o), _ptr(gate), gate.stride(0), _ptr(w), _ptr(out),
          out.stride(0), M, int(n_heads), N // n_heads, float(eps), 1 if gate_act == "silu" else 0, float(out_scale),
          _code(gate, "head_gated_rmsnorm"), _stream())
    return out


BLOCK_DIAG_MAX_TOKENS = 64      # up to this many tokens all blocks' products are one launch; beyond, a product per block


def block_diag_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [M, blocks * K] times a block-diagonal matrix given as w [blocks, N, K] -> float32 [M, blocks * N]: block b of the
    result is x's b-th K columns times w[b] transposed.  Few tokens: one kernel that reads every weight once (csrc/rglru.cu);
    many: the library's product, block by block."""
    _need_cuda(x, w, what="block_diag_linear")
    nb, N, Kb = w.shape
    M = x.shape[0]
    if x.dim() != 2 or x.shape[1] != nb * Kb or x.stride(1) != 1 or w.dtype != x.dtype or not w.is_contiguous():
        raise KernelError("block_diag_linear: the rows do not fit the blocks")
    out = torch.empty((M, nb * N), dtype=torch.float32, device=x.device)
    if M <= BLOCK_DIAG_MAX_TOKENS:
        _call(_fn("ti_block_diag_linear", [P, L, P, P, L, I, I, I, I, I, P]), _ptr(x), x.stride(0), _ptr(w), _ptr(out), out.stride(0), M,
              nb, N, Kb, _code(x, "block_diag_linear"), _stream())
        return out
    from . import gemm
    for b in range(nb):
        xb, wb, ob = x[:, b * Kb:(b + 1) * Kb], w[b], out[:, b * N:(b + 1) * N]
        gemm.run(xb, wb, ob, M, N, Kb, xb.stride(0), wb.stride(0))
    return out


SSD_SEGMENT = 256               # tokens of a segment; a step whose longest sequence brings two or more runs them in parallel


def ssd_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, rate: torch.Tensor, skip: Optional[torch.Tensor],
             n_heads: int, groups: int, n_state: int, vdim: int, state: torch.Tensor, state_offset: int, batch) -> torch.Tensor:
    """The Mamba-2 recurrence over every sequence's new tokens (csrc/ssd_scan.cu).  xbc [M, heads * vdim + 2 * groups *
    n_state]: x, B and C after their convolution and silu; dt_raw [M, heads] the raw step sizes (rows may be strided);
    dt_bias, rate (= exp(A_log)) and skip float32 [heads].  Returns float32 y [M, heads * vdim]; the state
    [heads, vdim, n_state] per slot is left as it is after the step's tokens.  Sequences that bring more than
    ``2 * SSD_SEGMENT`` tokens run as segments in parallel (three launches)."""
    _need_cuda(xbc, dt_raw, dt_bias, rate, skip, state, what="ssd_scan")
    M = xbc.shape[0]
    inner = n_heads * vdim
    if xbc.dim() != 2 or xbc.shape[1] != inner + 2 * groups * n_state or xbc.stride(1) != 1:
        raise KernelError("ssd_scan: x, B and C do not fit the heads, groups and state")
    if tuple(dt_raw.shape) != (M, n_heads) or dt_raw.dtype != xbc.dtype or dt_raw.stride(1) != 1:
        raise KernelError("ssd_scan: the step sizes must be [tokens, heads] of the tokens' type")
    for t, what in ((dt_bias, "step-size bias"), (rate, "rate"), (skip, "skip weight")):
        _vec(t, n_heads, f"ssd_scan: the {what}")
    base, stride = _state_part(state, state_offset, inner * n_state, "ssd_scan")
    y = torch.zeros((M, inner), dtype=torch.float32, device=xbc.device)         # rows that are nobody's stay zero
    seg = int(SSD_SEGMENT)
    n_seg = (batch.max_new + seg - 1) // seg if batch.max_new >= 2 * seg else 1
    scratch = decay = None
    if n_seg > 1:
        scratch = torch.empty((batch.n_seq * n_seg, inner * n_state), dtype=torch.float32, device=xbc.device)
        decay = torch.empty((batch.n_seq * n_seg, n_heads), dtype=torch.float32, device=xbc.device)
    _call(_fn("ti_ssd_scan", [P, L, P, L, P, P, P, P, L, P, P, P, I, I, I, I, I, I, I, P, P, I, P]),
          _ptr(xbc), xbc.stride(0), _ptr(dt_raw), dt_raw.stride(0), _ptr(dt_bias), _ptr(rate), _ptr(skip), base, stride, _ptr(y),
          _ptr(batch.cu_new), _ptr(batch.seq_slot), batch.n_seq, int(n_heads), int(groups), int(n_state), int(vdim), seg, n_seg,
          _ptr(scratch), _ptr(decay), _code(xbc, "ssd_scan"), _stream(), launches=3 if n_seg > 1 else 1)
    return y


def gate_group_rmsnorm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """y float32 [M, inner], z [M, inner] gate logits of the engine's type (rows may be strided), w float32 [inner] ->
    u / rms(u) * w with u = y * silu(z) and the root mean square taken over each of ``groups`` equal parts of the row, in
    the gate's type.  The gate comes before the norm."""
    _need_cuda(y, z, w, what="gate_group_rmsnorm")
    M, N = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or tuple(z.shape) != (M, N) or z.stride(1) != 1 or groups < 1 or N % groups:
        raise KernelError("gate_group_rmsnorm: y must be dense float32, the gate of its shape, the parts equal")
    _vec(w, N, "gate_group_rmsnorm: the weight")
    out = torch.empty((M, N), dtype=z.dtype, device=y.device)
    _call(_fn("ti_gate_group_rmsnorm", [P, P, L, P, P, I, I, I, F, I, P]), _ptr(y), _ptr(z), z.stride(0), _ptr(w), _ptr(out), M, N,
          int(groups), float(eps), _code(z, "gate_group_rmsnorm"), _stream())
    return out
