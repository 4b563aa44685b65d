"""RMS normalisation.

y_i = x_i * rsqrt(mean_j(x_j^2) + eps) * w_i, with the sum, the reciprocal square
root and the product in 32-bit and one rounding at the end; the weight multiplies
directly (no 1 + w).  Reference: src/decode.cu:99-125 (one token),
src/prefill.cu:74-94 (rows of a prompt).  The fused form adds the pending residual
first: the reference does that with a separate kernel (src/decode.cu:7-22) and a
copy (src/transformer.cpp:578-583).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import wide
from .base import BuildContext, Norm, ParamSpec, register_part


class RMSNorm(Norm):
    """``wide``: the hidden state it reads is a float32 stream whatever the engine's type, and what is pending on
    it may be up to three terms (kernels/wide.py); the normed rows come out in the engine's type."""

    def __init__(self, ctx: BuildContext, prefix: str, size: int, eps: float, name: str = "weight", wide: bool = False):
        self.size = int(size)
        self.eps = float(eps)
        self.weight_name = prefix + name
        self.weight: Optional[torch.Tensor] = None
        self.wide = bool(wide)
        self.out_dtype = ctx.dtype

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), role="norm", init="one_plus_normal")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.wide:
            return wide.add_norm_wide(x, None, self.weight, self.eps, self.out_dtype)
        return K.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, h: torch.Tensor, delta) -> torch.Tensor:
        if self.wide:
            return wide.add_norm_wide(h, delta, self.weight, self.eps, self.out_dtype)
        if isinstance(delta, tuple):
            raise ValueError("a pending sum of several terms needs a norm over a float32 stream (wide=True)")
        if delta is None:
            return K.rmsnorm(h, self.weight, self.eps)
        return K.add_rmsnorm(h, delta, self.weight, self.eps)

    def add_pending(self, h: torch.Tensor, delta):
        if self.wide:
            return self.add_forward(h, delta)
        pending = K.pending_norm(h, delta, self.weight, self.eps)
        return pending if pending is not None else self.add_forward(h, delta)

    def gather_add_forward(self, h: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        if self.wide:
            return wide.add_norm_wide(h, delta, self.weight, self.eps, self.out_dtype, rows=rows)
        return super().gather_add_forward(h, delta, rows)


register_part("norm", "rmsnorm", RMSNorm)


class StreamRMSNorm(Norm):
    """The norm that reads several float32 residual streams (kernels/hyper.py): y = rms(u) * w with
    u = sum_s read[s] X_s, after the update a sublayer left pending on X has been applied.  ``one_plus``: the stored
    weight lies around zero and 1 + w multiplies (formed once, in float32).  The weight is float32 whatever the
    engine's type; the normed rows come out in the engine's type."""

    def __init__(self, ctx: BuildContext, prefix: str, size: int, eps: float, name: str = "weight", streams: int = 1,
                 one_plus: bool = False):
        self.size, self.eps, self.streams = int(size), float(eps), int(streams)
        self.one_plus = bool(one_plus)
        self.weight_name = prefix + name
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype = ctx.dtype

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), role="norm", init="normal" if self.one_plus else "one_plus_normal")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.pop(self.weight_name).to(torch.float32)
        self.weight = (1.0 + w if self.one_plus else w).contiguous()

    def read_forward(self, X: torch.Tensor, pending, read: Optional[torch.Tensor]) -> torch.Tensor:
        """X takes ``pending`` (a kernels.hyper.StreamUpdate or None) in place; returns the norm of the streams read with ``read``."""
        from ..kernels import hyper
        return hyper.hyper_norm(X, pending, read, self.weight, self.eps, self.out_dtype, self.streams)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.read_forward(x, None, None)

    def add_forward(self, h: torch.Tensor, delta) -> torch.Tensor:
        return self.read_forward(h, delta, None)

    def gather_add_forward(self, h: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        """The norm of the sum of the streams of the rows ``rows``, the pending update included; h stays as it is."""
        from ..kernels import hyper
        return hyper.hyper_norm(h, delta, None, self.weight, self.eps, self.out_dtype, self.streams, rows=rows)


register_part("norm", "stream_rmsnorm", StreamRMSNorm)


class WideScalarRMSNorm(Norm):
    """RMS norm over a float32 residual stream whose weight is ONE number (``scalar``) or one per channel, in a design
    that norms a sublayer's output as well as its input: what is pending on the stream is a sublayer's output that still
    has to pass a norm of this kind (``pending(y)`` makes it, kernels.wide.PostNormed), and the next norm that reads the
    stream forms rmsnorm(y) * w_post, adds it in 32-bit and norms the sum, in one kernel.  The weight is float32 whatever
    the engine's type; the normed rows come out in the engine's type."""

    def __init__(self, ctx: BuildContext, prefix: str, size: int, eps: float, name: str = "weight", scalar: bool = True):
        self.size, self.eps, self.scalar = int(size), float(eps), bool(scalar)
        self.weight_name = prefix + name
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype = ctx.dtype

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec(() if self.scalar else (self.size,), role="norm", init="one_plus_normal", std=0.1)}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].to(torch.float32).reshape(-1).contiguous()

    def pending(self, y: torch.Tensor) -> "wide.PostNormed":
        """y as something that passes this norm before it is added to the stream."""
        return wide.PostNormed(y, self.weight, self.eps)

    def _check(self, delta) -> None:
        if delta is not None and not isinstance(delta, wide.PostNormed):
            raise ValueError("a stream with normed sublayer outputs takes what a norm's pending() made, nothing else")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return wide.post_norm_add_norm(x, None, self.weight, self.eps, self.out_dtype)

    def add_forward(self, h: torch.Tensor, delta) -> torch.Tensor:
        self._check(delta)
        return wide.post_norm_add_norm(h, delta, self.weight, self.eps, self.out_dtype)

    def gather_add_forward(self, h: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        self._check(delta)
        return wide.post_norm_add_norm(h, delta, self.weight, self.eps, self.out_dtype, rows=rows)


register_part("norm", "wide_scalar_rmsnorm", WideScalarRMSNorm)
