"""Plain, slow Bagasun: whole sequences, no cache, one function per mechanism.

The oracle of the Bagasun tests.  It shares no code with toyinfer_b200: the configuration is a
dict as config.json holds it, the weights a dict of tensors by checkpoint name, and every
mechanism is written with elementary torch operations in float64, token by token where the
mechanism is a recurrence.

The design in this file's notation (one row per token; W applies as W x; weights [out, in]):

* embedding:  x = E[token] * embedding.scale
* norm:       n(v; g) = v / sqrt(mean(v^2) + eps) * g, with g ONE number per norm
* layer:      x <- x + n(mixer(n(x; g1)); g1b);  x <- x + n(ff(n(x; g2)); g2b)  (ff may be absent).
              A layer with ``weights_of`` = j runs with layer j's tensors.
* sigmoid_attention ("attention"): q = Wq h + bq, k = Wk h + bk, v = Wv h + bv; q and k each normed
              over their WHOLE row (all heads together) with a weight of that length; head h reads kv
              head h // (H / G);  s_ij = q_i.k_j * scale - r1_h ln(1 + r2_h (i - j));  visible are
              the keys with 0 <= i - j < window;  w_ij = sigmoid(s_ij + pb_h), not normalised;
              o_i = sum_j w_ij v_j;  y = Wo o
* mamba2:     [z | x | B | C | dt] = Win h (inner, inner, G N, G N, heads);  (x, B, C) together go
              through a causal convolution per channel (taps, bias; last tap = current token) and
              silu;  dt <- softplus(dt + dt_bias);  per head (group = head // (heads / G)), with
              S [N, vdim] zero at the start:  S <- exp(-exp(A_log) dt) S + dt B x^T;
              y = S^T C + D x;  y <- y * silu(z);  y normed in ``norm_groups`` equal parts, times
              a weight [inner];  out = Wo y
* diff_attention ("attention_2"): q has H x 2 x dim rows, k has G x 2 x dim, v has G x vdim; two maps
              per head.  The first ``rot.dims`` elements of every map of q and k are rotated (pairs
              (i, i + dims/2), angle p f_i, f_i = base^(-2i/dims) rescaled for long contexts: kept
              where the wavelength is below original/high, divided by factor where it is above
              original/low, blended between).  Each map: causal softmax over the window of
              q.k * scale, times v -> a1, a2.  lambda = exp(lq1.lk1) - exp(lq2.lk2) + diff;
              o = a1 - lambda a2;  o <- o / sqrt(mean(o^2) + eps) * (1 - diff);
              o <- o * sigmoid(Wg h)_head;  y = Wo o
* feed-forward: Wdown (gelu_tanh(Wgate h) * (Wup h))
* output:     logits = head n(x; g_final)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

F64 = torch.float64


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    v = v.to(F64)
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(v: torch.Tensor, g, eps: float) -> torch.Tensor:
    return unit_rms(v, eps) * float(g)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gated_gelu_ff(h: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C]; taps [C, n] with the last column weighing the current row; zeros before row 0."""
    T, C = x.shape
    n = taps.shape[1]
    out = bias.to(F64).expand(T, C).clone()
    for j in range(n):
        back = n - 1 - j
        if back < T:
            out[back:] += x[:T - back] * taps[:, j]
    return out


def visible(m: dict, T: int) -> int:
    """How many positions a query sees, itself included: mask.size, or all when there is no mask."""
    return int(m["mask"]["size"]) if m.get("mask") else T


def sigmoid_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, width]; p: the mixer's tensors by their short names (q, q.b, k, ..., q.norm, k.norm, r1, r2, pb, o)."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window, scale = visible(m, T), float(m["scale"])
    zero = torch.zeros((), dtype=F64)
    q, k, v = (h @ p[n].T + p.get(n + ".b", zero) for n in ("q", "k", "v"))        # biases, the norm, the distance term and
    if "q.norm" in p:                                                              # the head's bias are each optional
        q, k = unit_rms(q, eps) * p["q.norm"], unit_rms(k, eps) * p["k.norm"]
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, vd)
    out = torch.zeros(T, H, vd, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            dist = torch.arange(i - lo, -1, -1, dtype=F64)                      # i - j for j = lo .. i
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale
            if "r1" in p:
                s = s - p["r1"][hd] * torch.log(1.0 + p["r2"][hd] * dist)
            out[i, hd] = sigmoid(s + (p["pb"][hd] if "pb" in p else 0.0)) @ v[lo:i + 1, g]
    return out.reshape(T, H * vd) @ p["o"].T


def scaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out.append(fi)
        elif wavelength > original / low:
            out.append(fi / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=F64)


def rotate_maps(x: torch.Tensor, dims: int, freqs: torch.Tensor, first_position: int = 0) -> torch.Tensor:
    """x [T, maps, dim]: the first ``dims`` elements of every map rotated by its row's position."""
    T = x.shape[0]
    half = dims // 2
    ang = (torch.arange(T, dtype=F64) + first_position)[:, None] * freqs[None, :]        # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], dim=-1)


def diff_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window, scale, diff = visible(m, T), float(m["scale"]), float(m["diff"])
    q = (h @ p["q"].T).view(T, H * 2, d)
    k = (h @ p["k"].T).view(T, G * 2, d)
    v = (h @ p["v"].T).view(T, G, vd)
    rot = m.get("rot")
    if rot:
        f = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_maps(q, rot["dims"], f), rotate_maps(k, rot["dims"], f)
    q, k = q.view(T, H, 2, d), k.view(T, G, 2, d)
    lam = math.exp(float((p["lq1"] * p["lk1"]).sum())) - math.exp(float((p["lq2"] * p["lk2"]).sum())) + diff
    gate = sigmoid(h @ p["g"].T) if "g" in p else torch.ones(T, H, dtype=F64)        # [T, H]; the gate is optional
    out = torch.zeros(T, H, vd, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            a = []
            for which in range(2):
                s = (k[lo:i + 1, g, which] @ q[i, hd, which]) * scale
                w = torch.softmax(s, dim=0)
                a.append(w @ v[lo:i + 1, g])
            o = a[0] - lam * a[1]
            out[i, hd] = unit_rms(o, eps) * (1.0 - diff) * gate[i, hd]
    return out.reshape(T, H * vd) @ p["o"].T


def mamba2(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    Hn, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hn * P
    zxbcdt = h @ p["in"].T
    z = zxbcdt[:, :inner]
    xbc = silu(causal_conv(zxbcdt[:, inner:2 * inner + 2 * G * N], p["conv"], p["conv.b"]))
    dt = softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + p["dt_bias"])                  # [T, heads]
    x = xbc[:, :inner].view(T, Hn, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    y = torch.zeros(T, Hn, P, dtype=F64)
    for hd in range(Hn):
        g = hd // (Hn // G)
        S = torch.zeros(N, P, dtype=F64)
        rate = math.exp(float(p["A_log"][hd]))
        for t in range(T):
            S = math.exp(-rate * float(dt[t, hd])) * S + float(dt[t, hd]) * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + p["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T


MIXERS = {"attention": sigmoid_attention, "attention_2": diff_attention, "mamba2": mamba2}


def layer_tensors(weights: Dict[str, torch.Tensor], layer: int, part: str) -> Dict[str, torch.Tensor]:
    pre = f"l{layer}.{part}."
    return {k[len(pre):]: v.to(F64) for k, v in weights.items() if k.startswith(pre)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """Returns (logits [T, vocab], the residual stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    x = weights["embed"].to(F64)[list(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    after = []
    for i, L in enumerate(cfg["layers"]):
        src = i
        while cfg["layers"][src].get("weights_of") is not None:          # a shared layer may name another shared one
            src = cfg["layers"][src]["weights_of"]
        g = lambda name: float(weights[f"l{src}.{name}"])
        mix = MIXERS[L["type"]](scalar_norm(x, g("norm1"), eps), layer_tensors(weights, src, "mix"), L["mixer"], eps)
        x = x + scalar_norm(mix, g("norm1b"), eps)
        if L.get("mlp") is not None:
            f = layer_tensors(weights, src, "mlp")
            ff = gated_gelu_ff(scalar_norm(x, g("norm2"), eps), f["gate"], f["up"], f["down"])
            x = x + scalar_norm(ff, g("norm2b"), eps)
        after.append(x.clone())
    logits = scalar_norm(x, float(weights["final.norm"]), eps) @ weights["head"].to(F64).T
    return logits, after
