"""Bolisun: the description of the model in terms of parts.

A pre-norm decoder over several float32 residual streams per token (hyper-connections: a sublayer reads a weighted sum of
the streams and its output is written back through a carry matrix and a write vector); the embedding's rows are scaled;
every mixer is two mixers side by side on the same input, softmax attention under a sliding window that keeps a
sequence's first positions visible (biases, per-head query/key norms, rotary positions on neighbouring pairs with
frequencies stretched for long contexts, grouped kv heads) and retention (linear attention with a fixed decay per head, a
float32 state, a weightless per-head norm and a silu gate), their outputs weighted; feed-forwards are dense with a clamped
gate, or mixtures of silu-gated experts under a softmax router with a choice correction and expert groups, beside a shared
expert; a layer may run with another layer's tensors and memory of its own; the head is the embedding table behind the
final norm of the streams' sum.  Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc1.*``,
``l<i>.hc2.*``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``.  Nothing here computes: the parts do.
"""
from __future__ import annotations

import json

from ..config.bolisun import BolisunConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec, ScheduleEntry


def describe_bolisun(cfg: BolisunConfig) -> ModelSpec:
    eps = cfg.eps
    streams = cfg.streams if cfg.streams is not None else 1
    norm = PartSpec("stream_rmsnorm", {"size": cfg.width, "eps": eps, "streams": streams})
    positions = {}
    own = [i for i in range(len(cfg.layers)) if cfg.weights_layer(i) == i]         # layers with tensors of their own
    layers = []
    for i in own:
        L = cfg.layers[i]
        m = L["mixer"]
        a, r = m["left"], m["right"]
        position = None
        rot = a.get("rot")
        if rot is not None:
            scaling = dict(rot["scaling"]) if rot.get("scaling") else None
            position = "rot:" + json.dumps([rot["dims"], rot["base"], scaling], sort_keys=True)
            positions.setdefault(position, PartSpec("rotary_half", {
                "dim": rot["dims"], "theta": rot["base"], "max_positions": cfg.max_positions, "scaling": scaling, "lazy": True,
                "pairing": "neighbours"}))
        mask = a.get("mask") or {}
        left = PartSpec("kept_window_attention", {
            "n_heads": a["heads"], "n_kv_heads": a["kv_heads"], "dim": a["dim"], "vdim": a["vdim"], "scale": a["scale"],
            "window": int(mask.get("size", 0)), "keep_first": int(mask.get("keep_first", 0)), "eps": eps, "position": position})
        right = PartSpec("retention", {"n_heads": r["heads"], "dim": r["dim"], "vdim": r["vdim"], "decay": list(r["decay"]), "eps": eps})
        mixer = PartSpec("side_by_side", {"left": left, "right": right, "left_scale": m["left_scale"], "right_scale": m["right_scale"]})
        f = L.get("mlp")
        ffn = None
        if f is not None and f["kind"] == "dense":
            ffn = PartSpec("gated_dense", {"intermediate_size": f["ff"], "act": "clamped_swish", "limit": f["limit"]})
        elif f is not None:
            g = f["router"].get("groups") or {}
            ffn = PartSpec("softmax_moe", {
                "n_experts": f["router"]["experts"], "top": f["router"]["top"], "intermediate_size": f["expert"]["ff"],
                "n_groups": int(g.get("count", 0)), "keep": int(g.get("keep", 0)), "scale": float(f["router"].get("scale", 1.0)),
                "shared_size": f["shared"]["ff"] if f.get("shared") else 0})
        block = PartSpec("hyper", {"norm": norm, "mixer": mixer, "feed_forward": ffn, "streams": streams,
                                   "connections": cfg.streams is not None, "layer_scale": False})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block))
    final = PartSpec(norm.kind, dict(norm.params, name="norm"))
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        layers=layers,
        final_norm=None,
        schedule=[ScheduleEntry(own.index(cfg.weights_layer(i))) for i in range(len(cfg.layers))],
        positions=positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "name": "embed", "wide": True, "copies": streams,
                                           "scale": cfg.embedding_scale}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "norm": final, "tied": True, "name": "head", "norm_prefix": "final."}),
        stop_token_ids=cfg.stop_token_ids,
    )


register_architecture("Bolisun", BolisunConfig, describe_bolisun)
