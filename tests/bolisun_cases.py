"""Small Bolisun configurations for the tests, each unlike the others in every size and option, and helpers to write a
model folder with random weights and to read it back for the plain implementation."""
from __future__ import annotations

import copy

import torch


def _left(heads, kv, dim, vdim, scale, window=None, keep=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    if rot:
        m["rot"] = rot
    return m


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _mix(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff, groups=None, scale=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        r["scale"] = scale
    f = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        f["shared"] = {"ff": shared}
    return f


_ROT_P = {"base": 1e4, "dims": 8}
_ROT_P_SCALED = {"base": 300.0, "dims": 12, "scaling": {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}}
_P0 = _mix(_left(6, 2, 16, 24, 0.25, window=40, keep=5, rot=_ROT_P), _right(3, 12, 20, [0.9, 0.97, 0.995]), 0.7, 1.3)
_P2 = _mix(_left(2, 1, 20, 12, 0.2, window=33, keep=9, rot=_ROT_P_SCALED), _right(2, 24, 8, [0.99, 0.8]), 1.1, 0.4)
_R0 = _mix(_left(3, 1, 12, 20, 0.3, window=64, keep=1), _right(1, 40, 40, [0.96]), 1.0, 1.0)

CASES = {
    # three streams; grouped kv heads (6 over 2, 2 over 1); values wider and narrower than keys; part of each head rotated,
    # once with stretched frequencies whose ramp lies inside the pairs; a dense and two expert feed-forwards (groups of
    # which not all stay; no groups; no shared expert) and a layer without; every layer once more with an earlier layer's tensors
    "P": {
        "architecture": "Bolisun", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5}, "streams": 3,
        "layers": [
            {"type": "parallel", "mixer": _P0, "mlp": _dense(40, 1.5)},
            {"type": "parallel", "mixer": _P0, "mlp": _moe(6, 2, 24, groups=(3, 2), scale=1.5, shared=16)},
            {"type": "parallel", "mixer": _P2, "mlp": _moe(5, 3, 16)},
            {"type": "parallel", "mixer": _P0, "mlp": _moe(6, 2, 24, groups=(3, 2), scale=1.5, shared=16), "weights_of": 1},
            {"type": "parallel", "mixer": _P2, "mlp": None},
            {"type": "parallel", "mixer": _P2, "mlp": None, "weights_of": 4},
            {"type": "parallel", "mixer": _P0, "mlp": _dense(40, 1.5), "weights_of": 0},
        ],
    },
    # one named stream; a head per kv head; the whole head rotated without stretching; no embedding key (scale one); windows
    # of a page and one, longer than any test sequence, and none at all (every earlier key); no kept positions, and more
    # kept positions than a window; one expert per token; all groups stay
    "Q": {
        "architecture": "Bolisun", "vocab": 310, "width": 96, "norm": {"eps": 1e-6}, "streams": 1,
        "layers": [
            {"type": "parallel", "mixer": _mix(_left(3, 3, 32, 16, 0.15, window=65, rot={"base": 500.0, "dims": 32}),
                                               _right(4, 8, 16, [0.5, 0.9, 0.99, 1.0]), 0.5, 2.0), "mlp": _moe(4, 1, 32, groups=(2, 2), shared=24)},
            {"type": "parallel", "mixer": _mix(_left(5, 5, 8, 8, 0.4, window=1000, keep=3), _right(2, 16, 4, [0.93, 0.97]), 1.5, 0.25),
             "mlp": _dense(72, 7.0)},
            {"type": "parallel", "mixer": _mix(_left(4, 2, 24, 24, 0.2, rot={"base": 1e6, "dims": 6}), _right(3, 20, 12, [0.999, 0.9, 0.95]), 1.0, 1.0),
             "mlp": None},
            {"type": "parallel", "mixer": _mix(_left(2, 2, 16, 32, 0.3, window=7, keep=20), _right(1, 64, 16, [0.98]), 0.9, 0.9),
             "mlp": _moe(8, 4, 8, groups=(4, 2), scale=0.5)},
        ],
    },
    # no streams key (a plain residual, no connection tensors); a chain of shared layers (3 -> 2 -> 0); no rotation; windows
    # of exactly a page; one kept position
    "R": {
        "architecture": "Bolisun", "vocab": 150, "width": 48, "norm": {"eps": 3e-6}, "embedding": {"scale": 0.5},
        "layers": [
            {"type": "parallel", "mixer": _R0, "mlp": _dense(32, 3.0)},
            {"type": "parallel", "mixer": _mix(_left(4, 4, 20, 12, 0.3, window=20, keep=2, rot={"base": 1e3, "dims": 20}),
                                               _right(2, 12, 24, [0.9, 0.99]), 0.3, 0.6), "mlp": _moe(3, 2, 20, shared=8)},
            {"type": "parallel", "mixer": _R0, "mlp": _dense(32, 3.0), "weights_of": 0},
            {"type": "parallel", "mixer": _R0, "mlp": _dense(32, 3.0), "weights_of": 2},
        ],
    },
    # heads of the sizes that real models use: keys and values of 128 and of 64, four streams, retention heads of 128 and 64
    "S": {
        "architecture": "Bolisun", "vocab": 120, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0}, "streams": 4,
        "layers": [
            {"type": "parallel", "mixer": _mix(_left(4, 2, 128, 128, 0.09, window=96, keep=4,
                                                     rot={"base": 1e6, "dims": 64, "scaling": {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}}),
                                               _right(2, 128, 64, [0.97, 0.999]), 0.9, 0.4), "mlp": _dense(64, 2.0)},
            {"type": "parallel", "mixer": _mix(_left(4, 1, 64, 64, 0.125, window=80, keep=70, rot={"base": 1e4, "dims": 64}),
                                               _right(2, 64, 128, [0.9, 0.95]), 1.2, 0.7), "mlp": _moe(8, 2, 32, groups=(2, 1), scale=2.0, shared=48)},
        ],
    },
    # sizes that are multiples of nothing: a width of 52 and a vocabulary of 97, heads of 10, 6, 5 and 3 elements, feed-forwards of
    # 11 and 9; two streams
    "T": {
        "architecture": "Bolisun", "vocab": 97, "width": 52, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5}, "streams": 2,
        "layers": [
            {"type": "parallel", "mixer": _mix(_left(3, 1, 10, 6, 0.3, window=11, keep=2, rot={"base": 100.0, "dims": 6}),
                                               _right(2, 5, 3, [0.9, 0.99]), 0.6, 0.75), "mlp": _dense(11, 2.0)},
            {"type": "parallel", "mixer": _mix(_left(2, 2, 6, 10, 0.4, window=70, keep=65), _right(3, 3, 7, [0.95, 0.8, 0.999]), 1.0, 1.5),
             "mlp": _moe(3, 2, 9, shared=7)},
        ],
    },
}
SEEDS = {"P": 35, "Q": 36, "R": 37, "S": 38, "T": 39}


def case(name: str) -> dict:
    return copy.deepcopy(CASES[name])


def write_folder(name: str, path: str) -> str:
    from toyinfer_b200.weights import write_model_folder
    write_model_folder(case(name), SEEDS[name], path)
    return path


def read_folder(path: str):
    """(weights by name, config dict) for the plain implementation, through its own reader."""
    from plain.qwen3_plain import read_config, read_weights
    return read_weights(path), read_config(path)


def prompts(name: str, lengths, seed: int = 0):
    g = torch.Generator().manual_seed(11000 + seed)
    v = CASES[name]["vocab"]
    return [torch.randint(0, v, (n,), generator=g).tolist() for n in lengths]


def assert_close_logits(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32 engine: 2e-5 + 2e-4 |want| against the float64 result: the sharp test, row by row.  bfloat16 engine: a
    row's error is its root mean square over the vocabulary (mean taken off) as a fraction of the row's spread.  Rounding
    alone leaves a few hundredths.  But a random router has close calls: where the bfloat16 choice scores of two experts
    fall the other way, that token runs another expert and its row is off by much more (later tokens feel it faintly
    through states and keys).  So the rows are judged together: half of them within 0.08, all but one in seven (or one)
    within 0.25, and none further off than a row's whole spread and a half.  (The same code runs in both types: what
    the float32 run passes is right.)"""
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-5, msg=lambda m: f"{what}: {m}")
        return
    spread = want.std(dim=-1) + 1e-3
    d = got - want
    err = (d - d.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt() / spread
    n = err.numel()
    report = f"{what}: row errors median {err.median():.3g}, max {err.max():.3g}, {int((err > 0.25).sum())} of {n} over 0.25"
    assert err.median() < 0.08, report
    assert int((err > 0.25).sum()) <= max(1, n // 7), report
    assert err.max() < 1.5, report
