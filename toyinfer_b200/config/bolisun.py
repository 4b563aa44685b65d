"""Configuration of the Bolisun decoder.

config.json names the design in ``architecture`` and gives: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``streams`` (how many residual streams a token has; with the key the layers carry connection tensors, without it there is
one plain stream), and ``layers``: per layer its ``type`` (``parallel``: windowed softmax attention beside retention), the
mixer's sizes and constants under ``mixer`` (``left``: heads, kv_heads, dim, vdim, scale, optionally ``mask`` {size,
keep_first} and ``rot`` {dims, base, optionally ``scaling`` {factor, original, fast, slow}}; ``right``: heads, dim, vdim,
decay (one per head); ``left_scale``, ``right_scale``), its feed-forward under ``mlp`` (null; ``kind`` dense with ``ff`` and
``limit``; or ``kind`` moe with ``expert`` {ff}, ``router`` {experts, top, optionally scale and ``groups`` {count, keep}} and
optionally ``shared`` {ff}), and optionally ``weights_of``: the index of the layer whose tensors this layer runs with (its
cache and state stay its own).  Every size and constant comes from there; nothing is assumed equal between layers.
"""
from __future__ import annotations

from typing import List

from .base import Key, ModelConfig
from .kadodra import _check_fields, _number


class BolisunConfig(ModelConfig):
    KEYS = {
        "architecture": Key("str"),
        "vocab": Key("int"),
        "width": Key("int"),
        "norm": Key("any"),
        "embedding": Key("any", required=False, default=None, nullable=True),
        "streams": Key("int", required=False, default=None, nullable=True),
        "layers": Key("any"),
        "max_positions": Key("int", required=False, default=131072),
        "stop_tokens": Key("int_or_list", required=False, default=()),
    }

    def _check_left(self, w: str, m, p: List[str]) -> None:
        if not _check_fields(w, m, {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float}, p):
            return
        if min(m["heads"], m["kv_heads"], m["dim"], m["vdim"]) < 1 or m["heads"] % m["kv_heads"]:
            p.append(f"{w}: {m['heads']} heads of {m['dim']} and {m['vdim']} elements over {m['kv_heads']} kv heads")
        mask = m.get("mask")
        if mask is not None:
            if not isinstance(mask, dict) or not isinstance(mask.get("size"), int) or mask["size"] < 1:
                p.append(f"{w}.mask.size: expected a positive integer")
            elif not isinstance(mask.get("keep_first", 0), int) or mask.get("keep_first", 0) < 0:
                p.append(f"{w}.mask.keep_first: expected an integer that is not negative")
        r = m.get("rot")
        if r is not None and _check_fields(w + ".rot", r, {"dims": int, "base": float}, p):
            if r["dims"] < 2 or r["dims"] % 2 or r["dims"] > m["dim"]:
                p.append(f"{w}.rot.dims: expected an even number from 2 to dim = {m['dim']}, got {r['dims']}")
            if r.get("scaling") is not None:
                _check_fields(w + ".rot.scaling", r["scaling"], {"factor": float, "original": int, "fast": float, "slow": float}, p)

    def _check_right(self, w: str, m, p: List[str]) -> None:
        if not _check_fields(w, m, {"heads": int, "dim": int, "vdim": int, "decay": list}, p):
            return
        if min(m["heads"], m["dim"], m["vdim"]) < 1:
            p.append(f"{w}: heads and their sizes must be positive")
        if len(m["decay"]) != m["heads"] or not all(_number(x) for x in m["decay"]):
            p.append(f"{w}.decay: expected {m['heads']} numbers, one per head")

    def _check_mlp(self, w: str, f, p: List[str]) -> None:
        if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
            p.append(f"{w}.kind: expected dense or moe")
        elif f["kind"] == "dense":
            if _check_fields(w, f, {"ff": int, "limit": float}, p) and (f["ff"] < 1 or not f["limit"] > 0):
                p.append(f"{w}: expected a positive ff and a positive limit")
        elif _check_fields(w + ".expert", f.get("expert"), {"ff": int}, p) and \
                _check_fields(w + ".router", f.get("router"), {"experts": int, "top": int}, p):
            r = f["router"]
            if not 1 <= r["top"] <= r["experts"]:
                p.append(f"{w}.router: top must lie in 1 .. experts")
            if not _number(r.get("scale", 1.0)):
                p.append(f"{w}.router.scale: not a number")
            g = r.get("groups")
            if g is not None and _check_fields(w + ".router.groups", g, {"count": int, "keep": int}, p):
                if g["count"] < 1 or r["experts"] % g["count"] or not 1 <= g["keep"] <= g["count"] \
                        or g["keep"] * (r["experts"] // g["count"]) < r["top"]:
                    p.append(f"{w}.router.groups: {r['experts']} experts in {g['count']} groups of which {g['keep']} stay do not "
                             f"give {r['top']} per token")
            if f.get("shared") is not None:
                _check_fields(w + ".shared", f["shared"], {"ff": int}, p)

    def validate(self) -> List[str]:
        p: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not isinstance(self.norm, dict) or not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            p.append("norm.eps: missing or not a positive number")
        if self.embedding is not None and (not isinstance(self.embedding, dict) or not _number(self.embedding.get("scale", 1.0))):
            p.append("embedding.scale: not a number")
        if self.streams is not None and not 1 <= self.streams <= 8:
            p.append(f"streams: expected 1 to 8, got {self.streams}")
        if not isinstance(self.layers, list) or not self.layers:
            p.append("layers: expected a non-empty list")
            return p
        for i, L in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") != "parallel":
                p.append(f"{w}.type: expected parallel")
                continue
            m = L.get("mixer")
            if _check_fields(w + ".mixer", m, {"left": dict, "right": dict, "left_scale": float, "right_scale": float}, p):
                self._check_left(w + ".mixer.left", m["left"], p)
                self._check_right(w + ".mixer.right", m["right"], p)
            if L.get("mlp") is not None:
                self._check_mlp(w + ".mlp", L["mlp"], p)
            j = L.get("weights_of")
            if j is not None and (not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(self.layers) or j == i):
                p.append(f"{w}.weights_of: expected the index of another layer")
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
