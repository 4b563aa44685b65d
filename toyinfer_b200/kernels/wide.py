"""A float32 residual stream beside activations of the engine's type (csrc/wide_residual.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Optional, Sequence, Tuple, Union

import torch

from . import KernelError, _call, _code, _i32, _need_cuda, _ptr, _stream
from .lib import declare

_fns = {}


def _fn(name, argtypes):
    f = _fns.get(name)
    if f is None:
        f = _fns[name] = declare(name, argtypes)
    return f


P, I, F = c_void_p, c_int, c_float
Pending = Union[None, torch.Tensor, Tuple[Optional[torch.Tensor], ...]]


def pending_terms(delta: Pending) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
    """(d0, d1, d2) of a pending sum: the stream becomes ((d0 + d1) + h) + d2."""
    if delta is None:
        return None, None, None
    if isinstance(delta, torch.Tensor):
        return delta, None, None
    terms = tuple(delta) + (None,) * (3 - len(delta))
    if len(terms) != 3:
        raise KernelError(f"a pending sum has at most three terms, got {len(delta)}")
    return terms


def embed_wide(table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, copies: int = 1) -> torch.Tensor:
    """float32 out[m] = table[ids[m]] * scale, ``copies`` times side by side ([M, copies * H])."""
    _need_cuda(table, ids, what="embed_wide")
    _i32(ids, "embed_wide ids")
    V, H = table.shape
    out = torch.empty((ids.numel(), int(copies) * H), dtype=torch.float32, device=table.device)
    _call(_fn("ti_embed_wide", [P, P, P, I, I, I, F, I, I, P]), _ptr(table), _ptr(ids), _ptr(out), ids.numel(), H, V,
          float(scale), int(copies), _code(table, "embed_wide"), _stream())
    return out


def add_norm_wide(h: torch.Tensor, delta: Pending, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                  rows: Optional[torch.Tensor] = None, want_out: bool = True) -> Optional[torch.Tensor]:
    """h (float32 [M, H]) takes the pending terms in place (without ``rows``); returns
    rmsnorm(h) * weight in ``out_dtype`` (the rounded sum itself when ``weight`` is None).  With
    ``rows`` only those rows are summed and normed and h is left as it is."""
    d0, d1, d2 = pending_terms(delta)
    _need_cuda(h, d0, d1, d2, weight, rows, what="add_norm_wide")
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_norm_wide: the stream must be a dense float32 [tokens, width] tensor")
    M, H = h.shape
    for d in (d0, d1, d2):
        if d is not None and (d.shape != h.shape or d.dtype != out_dtype or not d.is_contiguous()):
            raise KernelError(f"add_norm_wide: a pending term must be dense {out_dtype} of the stream's shape")
    w_f32 = 0
    if weight is not None:
        if weight.shape != (H,) or not weight.is_contiguous() or weight.dtype not in (out_dtype, torch.float32):
            raise KernelError(f"add_norm_wide: weight {tuple(weight.shape)} {weight.dtype} does not fit rows of {H}")
        w_f32 = 1 if weight.dtype == torch.float32 else 0
    R = M
    if rows is not None:
        _i32(rows, "add_norm_wide rows")
        R = rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=h.device) if want_out else None
    code = 0 if out_dtype == torch.float32 else 1
    _call(_fn("ti_add_norm_wide", [P, P, P, P, P, P, I, P, P, I, I, I, F, I, I, P]),
          _ptr(h), _ptr(d0), _ptr(d1), _ptr(d2), _ptr(rows), _ptr(weight), w_f32, _ptr(out), None, R, H, M, float(eps),
          0 if rows is not None else 1, code, _stream())
    return out


class PostNormed:
    """What a sublayer left pending on a float32 stream in a design that norms its sublayers' outputs too: the output
    ``y`` (engine type, [M, H]) and the norm it still has to pass (``weight`` float32, one number or H; ``eps``) before it
    is added.  ``post_norm_add_norm`` resolves it."""

    __slots__ = ("y", "weight", "eps")

    def __init__(self, y: torch.Tensor, weight: torch.Tensor, eps: float):
        self.y, self.weight, self.eps = y, weight, float(eps)


def _norm_weight(w: Optional[torch.Tensor], H: int, what: str) -> int:
    """The stride of a float32 norm weight of one number (0) or H (1)."""
    if w.dtype != torch.float32 or not w.is_contiguous() or w.numel() not in (1, H):
        raise KernelError(f"{what}: a norm weight must be dense float32 of 1 or {H} values")
    return 0 if w.numel() == 1 and H != 1 else 1 if w.numel() == H else 0


def post_norm_add_norm(h: torch.Tensor, pending: Optional[PostNormed], weight: Optional[torch.Tensor], eps: float,
                       out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """h (float32 [M, H]) takes rmsnorm(pending.y) * pending.weight in place (without ``rows``); returns
    rmsnorm(h) * weight in ``out_dtype`` (None when ``weight`` is None: only the sum is wanted).  With ``rows`` only those
    rows are summed and normed and h is left as it is."""
    y = pending.y if pending is not None else None
    wp = pending.weight if pending is not None else None
    _need_cuda(h, y, wp, weight, rows, what="post_norm_add_norm")
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("post_norm_add_norm: the stream must be a dense float32 [tokens, width] tensor")
    M, H = h.shape
    if y is not None and (y.shape != h.shape or y.dtype != out_dtype or not y.is_contiguous()):
        raise KernelError(f"post_norm_add_norm: the pending output must be dense {out_dtype} of the stream's shape")
    if pending is not None and weight is not None and abs(pending.eps - eps) > 0:
        raise KernelError("post_norm_add_norm: the two norms differ in eps")
    sp = _norm_weight(wp, H, "post_norm_add_norm") if wp is not None else 0
    sw = _norm_weight(weight, H, "post_norm_add_norm") if weight is not None else 0
    R = M
    if rows is not None:
        _i32(rows, "post_norm_add_norm rows")
        R = rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=h.device) if weight is not None else None
    _call(_fn("ti_post_norm_add_norm", [P, P, P, I, P, P, I, P, I, I, I, F, I, I, P]),
          _ptr(h), _ptr(y), _ptr(wp), sp, _ptr(rows), _ptr(weight), sw, _ptr(out), R, H, M,
          float(pending.eps if weight is None and pending is not None else eps), 0 if rows is not None else 1,
          0 if out_dtype == torch.float32 else 1, _stream())
    return out
