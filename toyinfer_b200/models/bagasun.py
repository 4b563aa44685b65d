"""Bagasun: the description of the model in terms of parts.

A decoder over a float32 residual stream whose sublayers are normed on the way in and on the way out, every norm with ONE
number as its weight; the embedding's rows are scaled; mixers are sliding-window attention with sigmoid weights and a
logarithmic distance term (biases, queries and keys normed over all heads at once, no rotation), differential
sliding-window attention (two softmax maps per head over shared values, rotary positions with banded frequency scaling,
a per-head output gate), or Mamba-2; feed-forwards are dense with a gelu gate; a layer may run with another layer's
tensors and memory of its own; the head is a matrix of its own behind the final norm.  Tensor names: ``embed``, ``head``,
``final.norm``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``.  Nothing here
computes: the parts do.
"""
from __future__ import annotations

import json

from ..config.bagasun import BagasunConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec, ScheduleEntry


def describe_bagasun(cfg: BagasunConfig) -> ModelSpec:
    eps = cfg.eps
    norm = PartSpec("wide_scalar_rmsnorm", {"size": cfg.width, "eps": eps, "scalar": True})
    positions = {}
    own = [i for i in range(len(cfg.layers)) if cfg.weights_layer(i) == i]         # layers with tensors of their own
    layers = []
    for i in own:
        L = cfg.layers[i]
        m = L["mixer"]
        window = int((m.get("mask") or {}).get("size", 0))
        if L["type"] == "attention":
            mixer = PartSpec("sigmoid_attention", {
                "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
                "window": window, "eps": eps})
        elif L["type"] == "attention_2":
            position = None
            rot = m.get("rot")
            if rot is not None:
                scaling = dict(rot["scaling"], kind="bands") if rot.get("scaling") else None
                position = "rot:" + json.dumps([rot["dims"], rot["base"], scaling], sort_keys=True)
                positions.setdefault(position, PartSpec("rotary_half", {
                    "dim": rot["dims"], "theta": rot["base"], "max_positions": cfg.max_positions, "scaling": scaling, "lazy": True}))
            mixer = PartSpec("diff_attention", {
                "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
                "window": window, "eps": eps, "diff": m["diff"], "position": position})
        else:
            mixer = PartSpec("mamba2", {"n_heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
                                        "conv": m["conv"], "norm_groups": m["norm_groups"], "eps": eps})
        f = L.get("mlp")
        ffn = PartSpec("gated_dense", {"intermediate_size": f["ff"], "act": "gelu_tanh"}) if f is not None else None
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("sandwich", {"norm": norm, "mixer": mixer, "feed_forward": ffn})))
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        layers=layers,
        final_norm=None,
        schedule=[ScheduleEntry(own.index(cfg.weights_layer(i))) for i in range(len(cfg.layers))],
        positions=positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "name": "embed", "wide": True, "scale": cfg.embedding_scale}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "norm": PartSpec(norm.kind, dict(norm.params, name="norm")), "tied": False,
                                 "name": "head", "norm_prefix": "final."}),
        stop_token_ids=cfg.stop_token_ids,
    )


register_architecture("Bagasun", BagasunConfig, describe_bagasun)
