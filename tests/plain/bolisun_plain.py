"""Plain, slow Bolisun: whole sequences, no cache, one function per mechanism.

The oracle of the Bolisun tests.  It shares no code with toyinfer_b200: the configuration is a
dict as config.json holds it, the weights a dict of tensors by checkpoint name, and every
mechanism is written with elementary torch operations in float64, token by token where the
mechanism is a recurrence.

The design in this file's notation (one row per token; W applies as W x; weights [out, in]):

* embedding:  X_s = E[token] * embedding.scale for each of the ``streams`` residual streams s
* norm:       n(v; w) = v / sqrt(mean(v^2) + eps) * w
* layer:      two sublayers (mixer; feed-forward, which may be absent), each with connection
              tensors a [S] ("in"), C [S, S] ("mix", [from, to]) and b [S] ("out"):
              u = sum_s a_s X_s;  y = sublayer(n(u; w));  X_t <- sum_s C_st X_s + b_t y, every t from the old X.
              A layer with ``weights_of`` = j runs with layer j's tensors.
* mixer:      left_scale * window_attention(h) + right_scale * retention(h), both on the same h
* window_attention: q = Wq h + bq [H, d], k = Wk h + bk [G, d], v = Wv h + bv [G, dv]; q and k normed per
              head over d with one weight [d] each; the first R = rot.dims elements of every head of q
              and k rotated in pairs (2i, 2i + 1) by the angle p g_i, where g_i is f_i = base^(-2i/R)
              blended with f_i / factor along a ramp between two pair indices, and cos and sin are
              multiplied by 0.1 ln(factor) + 1; head h reads kv head h // (H / G); s_ij = q_i.k_j * scale;
              key j is visible to query i when j <= i and (i - j < size or j < keep_first); softmax
              over the visible keys; y = Wo o + bo
* retention:  q = Wq h, k = Wk h * d^(-1/2) [H, d], v = Wv h [H, dv]; per head S [d, dv], zero at the
              start: S <- decay_h S + k v^T, o = S^T q; o / sqrt(mean(o^2) + eps) per head; times
              silu(Wg h); y = Wo o
* dense feed-forward: g = min(Wgate h, limit), u = clamp(Wup h, -limit, limit),
              y = Wdown (g * sigmoid(1.702 g) * (u + 1))
* experts:    z = Wr h; s = softmax(z); c = s + correction; experts in ``groups.count`` runs of neighbours,
              a run's score its largest c, only the ``groups.keep`` best runs stay in the choice; the
              ``top`` largest c among those; weights s_e / (sum of the chosen s + 1e-20) * router.scale;
              expert e: Wdown_e (silu(Wgate_e h) * (Wup_e h)); a shared expert of the same form is added
* output:     logits = E n(sum_s X_s; w_final)
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import torch

F64 = torch.float64


def rms_norm(v: torch.Tensor, w, eps: float) -> torch.Tensor:
    v = v.to(F64)
    out = v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)
    return out if w is None else out * w.to(F64)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def rotary_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """(angle per position for each of the dims / 2 pairs, the factor on cos and sin)."""
    R, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(R // 2, dtype=F64)
    f = base ** (-2.0 * i / R)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])
    where = lambda turns: R * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), R - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: elements (2i, 2i + 1), i < dims / 2, of every head turn by positions * g_i."""
    if not rot:
        return x
    R = int(rot["dims"])
    g, mag = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * g[None, :]                     # [T, R / 2]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:R:2], x[..., 1:R:2]
    out[..., 0:R:2] = a * c - b * s
    out[..., 1:R:2] = b * c + a * s
    return out


def visible(i: int, j: int, mask) -> bool:
    if j > i:
        return False
    if not mask:
        return True
    return i - j < int(mask["size"]) or j < int(mask.get("keep_first", 0))


def window_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).view(T, H, d)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, d)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, dv)
    q, k = rms_norm(q, p["q.norm"], eps), rms_norm(k, p["k.norm"], eps)
    pos = torch.arange(T)
    q, k = rotate_pairs(q, pos, m.get("rot")), rotate_pairs(k, pos, m.get("rot"))
    mask = m.get("mask")
    see = torch.tensor([[visible(i, j, mask) for j in range(T)] for i in range(T)])
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = torch.where(see, s, torch.full_like(s, -math.inf))
        w = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        o[:, hd] = (w / w.sum(dim=-1, keepdim=True)) @ v[:, g]
    return o.reshape(T, H * dv) @ p["o"].T + p["o.b"]


def retention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).view(T, H, d)
    k = (h @ p["k"].T).view(T, H, d) * d ** -0.5
    v = (h @ p["v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = float(m["decay"][hd]) * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_norm(o, None, eps).reshape(T, H * dv) * silu(h @ p["g"].T)
    return o @ p["o"].T


def sub(p: Dict[str, torch.Tensor], pre: str) -> Dict[str, torch.Tensor]:
    return {k[len(pre):]: v for k, v in p.items() if k.startswith(pre)}


def parallel_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    return float(m["left_scale"]) * window_attention(h, sub(p, "left."), m["left"], eps) \
        + float(m["right_scale"]) * retention(h, sub(p, "right."), m["right"], eps)


def clamped_ff(h: torch.Tensor, p: Dict[str, torch.Tensor], limit: float) -> torch.Tensor:
    g = torch.clamp(h @ p["gate"].T, max=limit)
    u = torch.clamp(h @ p["up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


def silu_expert(h: torch.Tensor, p: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def route(z: torch.Tensor, correction: torch.Tensor, r: dict) -> Tuple[List[int], torch.Tensor]:
    """One token's router logits -> (the chosen experts, their weights)."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.softmax(z.to(F64), dim=-1)
    c = s + correction.to(F64)
    groups = r.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        best = sorted(range(n), key=lambda g: (-float(c[g * per:(g + 1) * per].max()), g))[:keep]
        allowed = [e for e in range(E) if e // per in best]
    else:
        allowed = list(range(E))
    chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    w = s[chosen]
    return chosen, w / (w.sum() + 1e-20) * float(r.get("scale", 1.0))


def experts_ff(h: torch.Tensor, p: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    out = torch.zeros_like(h)
    z = h @ p["router"].T
    for t in range(h.shape[0]):
        chosen, w = route(z[t], p["correction"], f["router"])
        for e, we in zip(chosen, w):
            out[t] += we * silu_expert(h[t:t + 1], sub(p, f"e{e}."))[0]
    if f.get("shared"):
        out = out + silu_expert(h, sub(p, "shared."))
    return out


def feed_forward(h: torch.Tensor, p: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    if f["kind"] == "dense":
        return clamped_ff(h, p, float(f["limit"]))
    return experts_ff(h, p, f)


def layer_tensors(weights: Dict[str, torch.Tensor], layer: int, part: str) -> Dict[str, torch.Tensor]:
    pre = f"l{layer}.{part}."
    return {k[len(pre):]: v.to(F64) for k, v in weights.items() if k.startswith(pre)}


def read_streams(X: torch.Tensor, c: Dict[str, torch.Tensor]) -> torch.Tensor:
    """What a sublayer reads of the streams X [T, S, width]; without connection tensors there is one stream, read as it is."""
    return torch.einsum("s,nsw->nw", c["in"], X) if c else X[:, 0]


def connect(X: torch.Tensor, y: torch.Tensor, c: Dict[str, torch.Tensor]) -> torch.Tensor:
    """X [T, S, width] -> the streams after a sublayer's output y [T, width] has been written (a plain sum without
    connection tensors)."""
    if not c:
        return X + y[:, None, :]
    return torch.einsum("st,nsw->ntw", c["mix"], X) + c["out"][None, :, None] * y[:, None, :]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """Returns (logits [T, vocab], the sum of the streams after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams") or 1)
    E = weights["embed"].to(F64)
    x = E[list(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    X = x[:, None, :].repeat(1, S, 1)
    after = []
    for i, L in enumerate(cfg["layers"]):
        src = i
        while cfg["layers"][src].get("weights_of") is not None:
            src = cfg["layers"][src]["weights_of"]
        w = lambda name: weights[f"l{src}.{name}"].to(F64)
        c1 = layer_tensors(weights, src, "hc1")
        y = parallel_mixer(rms_norm(read_streams(X, c1), w("norm1"), eps), layer_tensors(weights, src, "mix"), L["mixer"], eps)
        X = connect(X, y, c1)
        if L.get("mlp") is not None:
            c2 = layer_tensors(weights, src, "hc2")
            y = feed_forward(rms_norm(read_streams(X, c2), w("norm2"), eps), layer_tensors(weights, src, "mlp"), L["mlp"])
            X = connect(X, y, c2)
        after.append(X.sum(dim=1))
    logits = rms_norm(X.sum(dim=1), weights["final.norm"], eps) @ E.T
    return logits, after
