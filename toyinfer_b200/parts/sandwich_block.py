"""A layer that norms every sublayer on the way in and on the way out.

h <- h + n1b(mixer(n1(h)));  h <- h + n2b(ffn(n2(h))), over a float32 stream h; the feed-forward (with its two norms)
may be absent.  A sublayer's output stays pending with the norm it has yet to pass, and the next norm that reads the
stream (this layer's n2, the next layer's n1, the head's) applies that norm, adds and norms again in one kernel
(parts/norms.py: ``wide_scalar_rmsnorm``), so the stream is read and written once per sublayer.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Block, BuildContext, ParamSpec, PartSpec, build_part, register_part


class SandwichBlock(Block):
    def __init__(self, ctx: BuildContext, prefix: str, norm: PartSpec, mixer: PartSpec,
                 feed_forward: Optional[PartSpec] = None, names: Optional[Dict[str, str]] = None):
        n = {"norm_in": "norm1", "norm_in_post": "norm1b", "norm_ff": "norm2", "norm_ff_post": "norm2b",
             "mixer": "mix.", "feed_forward": "mlp."}
        n.update(names or {})
        named = lambda key: build_part("norm", PartSpec(norm.kind, dict(norm.params, name=n[key])), ctx, prefix)
        self.norm_in, self.norm_in_post = named("norm_in"), named("norm_in_post")
        self.mixer = build_part("mixer", mixer, ctx, prefix + n["mixer"])
        self.feed_forward = self.norm_ff = self.norm_ff_post = None
        if feed_forward is not None:
            self.norm_ff, self.norm_ff_post = named("norm_ff"), named("norm_ff_post")
            self.feed_forward = build_part("feed_forward", feed_forward, ctx, prefix + n["feed_forward"])
        for norm_part in (self.norm_in_post, self.norm_ff_post):
            if norm_part is not None and not hasattr(norm_part, "pending"):
                raise ValueError(f"a sandwich block needs a norm that can stay pending on a sublayer's output; {norm.kind!r} cannot")
        self._children = tuple(c for c in (self.norm_in, self.norm_in_post, self.mixer, self.norm_ff, self.norm_ff_post,
                                           self.feed_forward) if c is not None)

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for c in self._children:
            out.update(c.param_specs())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for c in self._children:
            c.bind(tensors)

    def check_kernels(self, dtype) -> None:
        for c in self._children:
            c.check_kernels(dtype)

    @property
    def captures_start(self) -> bool:
        return bool(self.mixer.captures_start and (self.feed_forward is None or self.feed_forward.captures_start))

    def _mix(self, h, delta, batch, mem, shared):
        x = self.norm_in.add_forward(h, delta)                       # h takes what was pending; x = n1(h)
        return self.norm_in_post.pending(self.mixer.forward(x, batch, mem, shared))

    def _feed(self, h, a, batch):
        x = self.norm_ff.add_forward(h, a)
        return self.norm_ff_post.pending(self.feed_forward.forward(x, batch))

    def forward(self, h, delta, batch, mem, shared):
        trace = getattr(batch, "trace", None)
        if trace is not None and trace.active:
            with trace.range("layer.attn_block"):
                a = self._mix(h, delta, batch, mem, shared)
            if self.feed_forward is None:
                return h, a
            with trace.range("layer.mlp_block"):
                return h, self._feed(h, a, batch)
        a = self._mix(h, delta, batch, mem, shared)
        if self.feed_forward is None:
            return h, a
        return h, self._feed(h, a, batch)


register_part("block", "sandwich", SandwichBlock)
