"""What of the Bagasun design needs no device: the configuration's checks, which layer's tensors a layer runs with,
memory per layer run, tensor names, and the rescaled rotation frequencies."""
from __future__ import annotations

import pytest
import torch

from bagasun_cases import CASES, case
from plain import bagasun_plain as plain


def config(d):
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config.registry import architecture_of
    arch = architecture_of(d)
    return arch, arch.config_cls.from_dict(d)


@pytest.mark.parametrize("name", list(CASES))
def test_shared_layers_have_no_tensors_but_memory_of_their_own(name):
    from toyinfer_b200.parts.model import DecoderModel
    d = case(name)
    arch, cfg = config(d)
    model = DecoderModel(arch.describe(cfg), torch.float32, "cpu")
    own = [i for i, L in enumerate(d["layers"]) if "weights_of" not in L]
    assert len(model.blocks) == len(own)

    def source(i):
        while "weights_of" in d["layers"][i]:
            i = d["layers"][i]["weights_of"]
        return i
    assert [own[e.layer] for e in model.schedule] == [source(i) for i in range(len(d["layers"]))]
    reqs = model.memory_requests()
    assert len(reqs) == len(d["layers"]) and all(r is not None for r in reqs)
    names = set(model.param_specs())
    for i, L in enumerate(d["layers"]):
        assert any(n.startswith(f"l{i}.") for n in names) == ("weights_of" not in L)
        if "weights_of" not in L:
            assert (f"l{i}.mlp.gate" in names) == (L["mlp"] is not None) and (f"l{i}.norm2b" in names) == (L["mlp"] is not None)
            assert model.param_specs()[f"l{i}.norm1"].shape == ()
    assert {"embed", "head", "final.norm"} <= names


def test_tensor_names_and_shapes_of_each_mixer():
    from toyinfer_b200.parts.model import DecoderModel
    arch, cfg = config(case("U"))
    s = DecoderModel(arch.describe(cfg), torch.float32, "cpu").param_specs()
    shape = lambda n: tuple(s[n].shape)
    assert shape("l0.mix.q") == (96, 64) and shape("l0.mix.q.b") == (96,) and shape("l0.mix.k.norm") == (32,) and shape("l0.mix.v") == (48, 64)
    assert shape("l0.mix.r1") == shape("l0.mix.r2") == shape("l0.mix.pb") == (6,) and shape("l0.mix.o") == (64, 144)
    assert shape("l1.mix.in") == (2 * 48 + 2 * 3 * 16 + 6, 64) and shape("l1.mix.conv") == (48 + 96, 3) and shape("l1.mix.conv.b") == (144,)
    assert shape("l1.mix.dt_bias") == shape("l1.mix.A_log") == shape("l1.mix.D") == (6,) and shape("l1.mix.norm") == (48,)
    assert shape("l2.mix.q") == (2 * 2 * 24, 64) and shape("l2.mix.k") == (48, 64) and shape("l2.mix.v") == (40, 64)
    assert shape("l2.mix.lq1") == (24,) and shape("l2.mix.g") == (2, 64) and shape("l2.mix.o") == (64, 80)
    assert "l2.mix.q.b" not in s and "l0.mix.g" not in s


def test_configuration_problems_are_all_reported():
    from toyinfer_b200.config.base import ConfigError
    d = case("U")
    d["layers"][0]["mixer"]["kv_heads"] = 4                  # 6 heads over 4
    d["layers"][1]["mixer"]["norm_groups"] = 5               # 48 channels in 5 parts
    d["layers"][2]["mixer"]["rot"]["dims"] = 26              # more than a map holds
    d["layers"][3]["weights_of"] = 0                         # a layer of another type
    d["layers"][4]["type"] = "nothing"
    d["layers"][5]["mlp"] = {"kind": "sparse"}
    with pytest.raises(ConfigError) as e:
        config(d)
    msg = str(e.value)
    for piece in ("6 heads over 4", "48 channels", "rot.dims", "layers[3].weights_of", "layers[4].type", "layers[5].mlp"):
        assert piece in msg, (piece, msg)
    d = case("W")
    d["layers"][0]["weights_of"] = 3                          # 0 -> 3 -> 2 -> 0
    with pytest.raises(ConfigError) as e:
        config(d)
    assert "never ends" in str(e.value)


@pytest.mark.parametrize("dims,base,scaling", [
    (24, 1e4, None),
    (8, 500.0, {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 64}),
    (64, 5e5, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}),
    (32, 1e6, {"factor": 2.0, "low": 1.0, "high": 1.0, "original": 256}),        # no band between the two
])
def test_rotation_tables_follow_the_banded_rule(dims, base, scaling):
    from toyinfer_b200.parts.rope import rotary_tables
    f = plain.scaled_frequencies(dims, base, scaling)
    cos, sin = rotary_tables(dims, base, 300, dict(scaling, kind="bands") if scaling else None)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    torch.testing.assert_close(cos.double(), torch.cos(ang), rtol=0, atol=1e-7)
    torch.testing.assert_close(sin.double(), torch.sin(ang), rtol=0, atol=1e-7)
    if scaling and scaling["high"] != scaling["low"]:
        plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        kept, slowed = (f == plainf), torch.isclose(f, plainf / scaling["factor"], rtol=1e-12)
        assert kept.any() and slowed.any()                     # both ends of the rule occur in these cases


def test_lambda_of_a_differential_layer_is_one_number_formed_at_load_time():
    from toyinfer_b200.parts import BuildContext, PartSpec, build_part
    ctx = BuildContext(dtype=torch.float32, device=torch.device("cpu"), hidden_size=32)
    m = build_part("mixer", PartSpec("diff_attention", dict(n_heads=2, n_kv_heads=1, dim=8, vdim=8, scale=0.3, window=5, eps=1e-5,
                                                             diff=0.35, position=None)), ctx, "a.")
    g = torch.Generator().manual_seed(3)
    t = {n: torch.randn(s.shape, generator=g) * 0.3 for n, s in m.param_specs().items()}
    want = float(torch.exp((t["a.lq1"].double() * t["a.lk1"].double()).sum()) - torch.exp((t["a.lq2"].double() * t["a.lk2"].double()).sum()) + 0.35)
    m.bind(dict(t))
    assert abs(m.lam - want) < 1e-12
