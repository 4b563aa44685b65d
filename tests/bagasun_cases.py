"""Small Bagasun configurations for the tests, each unlike the others in every size and option, and helpers to write a
model folder with random weights and to read it back for the plain implementation."""
from __future__ import annotations

import copy

import torch


def _sig(heads, kv, dim, vdim, scale, window=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return m


def _diff(heads, kv, dim, vdim, scale, diff, window=None, rot=None):
    m = _sig(heads, kv, dim, vdim, scale, window)
    m["diff"] = diff
    if rot:
        m["rot"] = rot
    return m


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _ff(n):
    return {"kind": "dense", "ff": n}


CASES = {
    # every mixer once and each once more with an earlier layer's tensors; grouped heads (6 over 2, 2 over 1); values wider
    # than keys; the whole map rotated (rot.dims == dim), no frequency scaling; a layer without a feed-forward; three
    # state groups and three norm parts
    "U": {
        "architecture": "Bagasun", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
        "layers": [
            {"type": "attention", "mixer": _sig(6, 2, 16, 24, 0.25, window=40), "mlp": _ff(40)},
            {"type": "mamba2", "mixer": _ssm(6, 8, 16, 3, 3, 3), "mlp": None},
            {"type": "attention_2", "mixer": _diff(2, 1, 24, 40, 0.2, 0.3, window=33, rot={"base": 1e4, "dims": 24}), "mlp": _ff(72)},
            {"type": "mamba2", "mixer": _ssm(6, 8, 16, 3, 3, 3), "mlp": None, "weights_of": 1},
            {"type": "attention_2", "mixer": _diff(2, 1, 24, 40, 0.2, 0.3, window=33, rot={"base": 1e4, "dims": 24}), "mlp": _ff(72),
             "weights_of": 2},
            {"type": "attention", "mixer": _sig(6, 2, 16, 24, 0.25, window=40), "mlp": _ff(40), "weights_of": 0},
        ],
    },
    # no shared layers; a head per kv head (groups of one); one state group, one norm part, a state that is no multiple of
    # eight, two taps; part of each map rotated with scaled frequencies whose bands all occur; windows longer than a page
    "V": {
        "architecture": "Bagasun", "vocab": 310, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
        "layers": [
            {"type": "mamba2", "mixer": _ssm(3, 20, 44, 1, 2, 1), "mlp": _ff(24)},
            {"type": "attention_2", "mixer": _diff(3, 3, 32, 16, 0.15, 0.8, window=100,
                                                   rot={"base": 500.0, "dims": 8, "scaling": {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 64}}),
             "mlp": _ff(80)},
            {"type": "attention", "mixer": _sig(5, 5, 8, 8, 0.4, window=70), "mlp": None},
            {"type": "mamba2", "mixer": _ssm(8, 4, 8, 8, 5, 2), "mlp": _ff(56)},
        ],
    },
    # a chain of shared layers (3 -> 2 -> 0); no embedding key (scale one); attention without a mask (every earlier key) and
    # without rotation; windows of exactly a page and of one position more
    "W": {
        "architecture": "Bagasun", "vocab": 150, "width": 48, "norm": {"eps": 3e-6},
        "layers": [
            {"type": "attention_2", "mixer": _diff(3, 1, 12, 20, 0.3, 0.5, window=64), "mlp": _ff(32)},
            {"type": "attention", "mixer": _sig(2, 2, 20, 12, 0.3, window=65), "mlp": _ff(24)},
            {"type": "attention_2", "mixer": _diff(3, 1, 12, 20, 0.3, 0.5, window=64), "mlp": _ff(32), "weights_of": 0},
            {"type": "attention_2", "mixer": _diff(3, 1, 12, 20, 0.3, 0.5, window=64), "mlp": _ff(32), "weights_of": 2},
            {"type": "attention", "mixer": _sig(4, 1, 16, 16, 0.2), "mlp": None},
            {"type": "mamba2", "mixer": _ssm(2, 16, 24, 2, 1, 4), "mlp": _ff(16)},
        ],
    },
    # heads of the sizes that real models use: keys of 128 with values of 64 and the other way round, a state of 128
    "X": {
        "architecture": "Bagasun", "vocab": 120, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
        "layers": [
            {"type": "attention", "mixer": _sig(4, 2, 128, 64, 0.09, window=96), "mlp": _ff(64)},
            {"type": "mamba2", "mixer": _ssm(2, 64, 128, 2, 4, 2), "mlp": _ff(48)},
            {"type": "attention_2", "mixer": _diff(4, 2, 64, 128, 0.125, 0.2, window=80,
                                                   rot={"base": 1e6, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}}),
             "mlp": None},
        ],
    },
}
SEEDS = {"U": 25, "V": 26, "W": 27, "X": 28}


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
    g = torch.Generator().manual_seed(9000 + seed)
    v = CASES[name]["vocab"]
    return [torch.randint(0, v, (n,), generator=g).tolist() for n in lengths]


def assert_close_logits(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32 engine: 2e-5 + 2e-4 |want| against the float64 result, element by element.  bfloat16 engine: a row's error
    is its root mean square over the vocabulary (mean taken off) as a fraction of the row's spread; rounding of
    activations and of the cached keys and values leaves a few hundredths, and no row may be further off than 0.15."""
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-5, msg=lambda m: f"{what}: {m}")
        return
    spread = want.std(dim=-1) + 1e-3
    d = got - want
    err = (d - d.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt() / spread
    report = f"{what}: row errors median {err.median():.3g}, max {err.max():.3g}"
    assert err.median() < 0.06, report
    assert err.max() < 0.15, report
