"""Configuration of the Bagasun decoder.

config.json names the design in ``architecture`` and gives: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, and
``layers``: per layer its ``type`` (``attention``: sigmoid-weighted sliding-window attention; ``attention_2``: differential
sliding-window attention with rotary positions; ``mamba2``), the mixer's sizes and constants under ``mixer``, its
feed-forward under ``mlp`` (null, or ``kind`` dense with ``ff``), and optionally ``weights_of``: the index of the layer
whose tensors this layer runs with (its cache or state stays its own).  Every size and constant comes from there;
nothing is assumed equal between layers.
"""
from __future__ import annotations

from typing import List

from .base import Key, ModelConfig
from .kadodra import _check_fields, _number

MIXER_KEYS = {
    "attention": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float},
    "attention_2": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "diff": float},
    "mamba2": {"heads": int, "vdim": int, "state": int, "groups": int, "conv": int, "norm_groups": int},
}


class BagasunConfig(ModelConfig):
    KEYS = {
        "architecture": Key("str"),
        "vocab": Key("int"),
        "width": Key("int"),
        "norm": Key("any"),
        "embedding": Key("any", required=False, default=None, nullable=True),
        "layers": Key("any"),
        "max_positions": Key("int", required=False, default=131072),
        "stop_tokens": Key("int_or_list", required=False, default=()),
    }

    def validate(self) -> List[str]:
        p: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not isinstance(self.norm, dict) or not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            p.append("norm.eps: missing or not a positive number")
        if self.embedding is not None and (not isinstance(self.embedding, dict) or not _number(self.embedding.get("scale", 1.0))):
            p.append("embedding.scale: not a number")
        if not isinstance(self.layers, list) or not self.layers:
            p.append("layers: expected a non-empty list")
            return p
        for i, L in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_KEYS:
                p.append(f"{w}.type: expected one of {sorted(MIXER_KEYS)}")
                continue
            m = L.get("mixer")
            if not _check_fields(w + ".mixer", m, MIXER_KEYS[L["type"]], p):
                continue
            if L["type"] == "mamba2":
                if m["groups"] < 1 or m["heads"] % m["groups"]:
                    p.append(f"{w}.mixer: {m['heads']} heads over {m['groups']} groups")
                if m["norm_groups"] < 1 or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    p.append(f"{w}.mixer: {m['heads'] * m['vdim']} channels do not cut into {m['norm_groups']} equal norm parts")
                if not 1 <= m["conv"] <= 8:
                    p.append(f"{w}.mixer.conv: expected 1 to 8 taps, got {m['conv']}")
                if m["state"] < 1:
                    p.append(f"{w}.mixer.state: expected a positive size")
            else:
                if m["kv_heads"] < 1 or m["heads"] % m["kv_heads"]:
                    p.append(f"{w}.mixer: {m['heads']} heads over {m['kv_heads']} kv heads")
                mask = m.get("mask")
                if mask is not None and (not isinstance(mask, dict) or not isinstance(mask.get("size"), int) or mask["size"] < 1):
                    p.append(f"{w}.mixer.mask.size: expected a positive integer")
            if L["type"] == "attention_2" and m.get("rot") is not None:
                r = m["rot"]
                if _check_fields(w + ".mixer.rot", r, {"dims": int, "base": float}, p):
                    if r["dims"] < 2 or r["dims"] % 2 or r["dims"] > m["dim"]:
                        p.append(f"{w}.mixer.rot.dims: expected an even number from 2 to dim = {m['dim']}, got {r['dims']}")
                    if r.get("scaling") is not None:
                        _check_fields(w + ".mixer.rot.scaling", r["scaling"], {"factor": float, "low": float, "high": float,
                                                                                 "original": int}, p)
            f = L.get("mlp")
            if f is not None and (not isinstance(f, dict) or f.get("kind") != "dense" or not isinstance(f.get("ff"), int) or f["ff"] < 1):
                p.append(f"{w}.mlp: expected null or kind dense with a positive ff")
            j = L.get("weights_of")
            if j is not None:
                if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(self.layers) or j == i:
                    p.append(f"{w}.weights_of: expected the index of another layer")
                elif isinstance(self.layers[j], dict) and self.layers[j].get("type") != L["type"]:
                    p.append(f"{w}.weights_of: layer {j} is of another type")
        if not p:
            for i in range(len(self.layers)):
                seen, j = set(), i
                while self.layers[j].get("weights_of") is not None:
                    if j in seen:
                        p.append(f"layers[{i}].weights_of: the chain of shared weights never ends")
                        break
                    seen.add(j)
                    j = self.layers[j]["weights_of"]
        return p

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float((self.embedding or {}).get("scale", 1.0))

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs with (itself, unless ``weights_of`` says otherwise)."""
        while self.layers[i].get("weights_of") is not None:
            i = self.layers[i]["weights_of"]
        return i

    @property
    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)
