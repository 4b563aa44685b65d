"""Linear attention with a per-head decay and a state per sequence, and the gated norm after it
(csrc/lightning.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import KernelError, _call, _code, _need_cuda, _ptr, _stream
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float
CHUNK = 64                 # tokens per chunk of the chunked form (csrc/lightning.cu)
CHUNKED_FROM = 32          # new tokens of one sequence from which a step runs the chunked form (three launches)


def mix(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, batch,
        act: str = "silu", k_scale: float = 1.0) -> torch.Tensor:
    """q, k [M, heads, dim] and v [M, heads, vdim] as projected: they pass ``act`` ("silu" or "none") as they enter the
    recurrence, and k is then multiplied by ``k_scale``; ``state`` float32 [slots, heads, dim, vdim] is read at each
    sequence's slot and left as it is after the step's tokens.  Returns float32 [M, heads * vdim]."""
    if act not in ("silu", "none"):
        raise KernelError(f"lightning: unknown entry function {act!r}")
    a = 1 if act == "silu" else 0
    _need_cuda(q, k, v, state, decay, what="lightning")
    M, nh, dim = q.shape
    vdim = v.shape[2]
    if k.shape != q.shape or v.shape[:2] != (M, nh) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("lightning: q, k and v do not fit together")
    for t in (q, k, v):
        if t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise KernelError("lightning: heads of a token must be dense")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (nh, dim, vdim) or not state.is_contiguous():
        raise KernelError("lightning: the state must be float32 [slots, heads, dim, vdim]")
    if decay.dtype != torch.float32 or decay.shape != (nh,):
        raise KernelError("lightning: the decays must be float32 [heads]")
    o = torch.empty((M, nh * vdim), dtype=torch.float32, device=q.device)
    code = _code(q, "lightning")
    if batch.max_new >= CHUNKED_FROM:
        n_chunks = (batch.n_tok + CHUNK - 1) // CHUNK + batch.n_seq
        U = torch.empty((n_chunks, nh, dim, vdim), dtype=torch.float32, device=q.device)
        _call(_fn("ti_lightning_chunked", [P, P, P, L, L, L, P, P, P, P, P, P, I, I, I, I, I, I, F, I, P]),
              _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(o), _ptr(state), _ptr(U), _ptr(decay),
              _ptr(batch.cu_new), _ptr(batch.seq_slot), batch.n_seq, n_chunks, nh, dim, vdim, a, float(k_scale), code, _stream(), launches=3)
    else:
        _call(_fn("ti_lightning_scan", [P, P, P, L, L, L, P, P, P, P, P, I, I, I, I, I, F, I, P]),
              _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(o), _ptr(state), _ptr(decay),
              _ptr(batch.cu_new), _ptr(batch.seq_slot), batch.n_seq, nh, dim, vdim, a, float(k_scale), code, _stream())
    return o


def gated_rmsnorm(o: torch.Tensor, g: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """rms(o) * w * sigmoid(g): o float32 [M, N], g [M, N] (rows may be strided) of the engine's type, w float32 [N]."""
    _need_cuda(o, g, w, what="gated_rmsnorm")
    M, N = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or g.shape != (M, N) or g.stride(1) != 1:
        raise KernelError("gated_rmsnorm: o must be dense float32 and g of its shape")
    if w.dtype != torch.float32 or w.shape != (N,) or not w.is_contiguous():
        raise KernelError("gated_rmsnorm: the weight must be float32 [N]")
    out = torch.empty((M, N), dtype=g.dtype, device=o.device)
    _call(_fn("ti_gated_rmsnorm", [P, P, L, P, P, I, I, F, I, P]), _ptr(o), _ptr(g), g.stride(0), _ptr(w), _ptr(out), M, N,
          float(eps), _code(g, "gated_rmsnorm"), _stream())
    return out
