"""What of the Bolisun design needs no device: the configuration's checks, which layer's tensors a layer runs with, the
two memories of every layer run, tensor names, the stretched rotation frequencies, and a tuple of requests in the cache."""
from __future__ import annotations

import pytest
import torch

from bolisun_cases import CASES, case
from plain import bolisun_plain as plain


def config(d):
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config.registry import architecture_of
    arch = architecture_of(d)
    return arch, arch.config_cls.from_dict(d)


@pytest.mark.parametrize("name", list(CASES))
def test_shared_layers_have_no_tensors_but_two_memories_of_their_own(name):
    from toyinfer_b200.parts import KVRequest, StateRequest
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
    assert len(reqs) == len(d["layers"])
    for r, L in zip(reqs, d["layers"]):
        a, b = L["mixer"]["left"], L["mixer"]["right"]
        assert isinstance(r, tuple) and isinstance(r[0], KVRequest) and isinstance(r[1], StateRequest)
        assert (r[0].n_kv_heads, r[0].head_dim, r[0].value_dim or r[0].head_dim) == (a["kv_heads"], a["dim"], a["vdim"])
        assert tuple(r[1].shape) == (b["heads"], b["dim"], b["vdim"])
    names = set(model.param_specs())
    for i, L in enumerate(d["layers"]):
        assert any(n.startswith(f"l{i}.") for n in names) == ("weights_of" not in L)
        if "weights_of" not in L:
            assert (f"l{i}.norm2" in names) == (L["mlp"] is not None)
            assert (f"l{i}.hc1.mix" in names) == ("streams" in d) and (f"l{i}.hc2.in" in names) == ("streams" in d and L["mlp"] is not None)
    assert {"embed", "final.norm"} <= names and "head" not in names


def test_tensor_names_and_shapes():
    from toyinfer_b200.parts.model import DecoderModel
    arch, cfg = config(case("P"))
    s = DecoderModel(arch.describe(cfg), torch.float32, "cpu").param_specs()
    shape = lambda n: tuple(s[n].shape)
    assert shape("l0.mix.left.q") == (96, 64) and shape("l0.mix.left.q.b") == (96,) and shape("l0.mix.left.k.norm") == (16,)
    assert shape("l0.mix.left.v") == (48, 64) and shape("l0.mix.left.o") == (64, 144) and shape("l0.mix.left.o.b") == (64,)
    assert shape("l0.mix.right.q") == shape("l0.mix.right.k") == (36, 64) and shape("l0.mix.right.v") == shape("l0.mix.right.g") == (60, 64)
    assert shape("l0.mix.right.o") == (64, 60) and "l0.mix.right.q.b" not in s and "l0.mix.right.norm" not in s
    assert shape("l0.mlp.gate") == (40, 64) and shape("l0.hc1.mix") == (3, 3) and shape("l0.hc2.out") == (3,)
    assert shape("l1.mlp.e5.up") == (24, 64) and shape("l1.mlp.router") == (6, 64) and shape("l1.mlp.correction") == (6,)
    assert shape("l1.mlp.shared.down") == (64, 16) and "l2.mlp.shared.gate" not in s and shape("l2.mlp.e4.down") == (64, 16)
    assert "l4.norm2" not in s and "l4.hc2.in" not in s and "l3.norm1" not in s


def test_configuration_problems_are_all_reported():
    from toyinfer_b200.config.base import ConfigError
    d = case("P")
    d["layers"][0]["mixer"]["left"]["kv_heads"] = 4                   # 6 heads over 4
    d["layers"][1]["mixer"]["right"]["decay"] = [0.9]                 # one decay for three heads
    d["layers"][2]["mixer"]["left"]["rot"]["dims"] = 22               # more than a head holds
    d["layers"][1]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}   # 6 experts do not cut into 4 groups
    d["layers"][4]["type"] = "nothing"
    d["layers"][6]["weights_of"] = 6
    d["layers"][0]["mlp"] = {"kind": "dense", "ff": 40}                 # no limit
    with pytest.raises(ConfigError) as e:
        config(d)
    msg = str(e.value)
    for piece in ("6 heads", "decay", "rot.dims", "router.groups", "layers[4].type", "layers[6].weights_of", "layers[0].mlp.limit"):
        assert piece in msg, (piece, msg)
    d = case("R")
    d["layers"][0]["weights_of"] = 3                          # 0 -> 3 -> 2 -> 0
    with pytest.raises(ConfigError) as e:
        config(d)
    assert "never ends" in str(e.value)


@pytest.mark.parametrize("rot", [
    {"dims": 24, "base": 1e4},
    {"dims": 12, "base": 300.0, "scaling": {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}},
    {"dims": 64, "base": 1e6, "scaling": {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}},
    {"dims": 6, "base": 50.0, "scaling": {"factor": 2.0, "original": 16, "fast": 2.0, "slow": 0.5}},         # the ramp spans all three pairs
])
def test_rotation_tables_against_the_rule(rot):
    from toyinfer_b200.parts.rope import rotary_tables
    cos, sin = rotary_tables(rot["dims"], rot["base"], 300, rot.get("scaling"))
    f, mag = plain.rotary_frequencies(rot)
    pos = torch.arange(300, dtype=torch.float64)
    torch.testing.assert_close(cos.double(), torch.cos(pos[:, None] * f) * mag, rtol=0, atol=1e-6)
    torch.testing.assert_close(sin.double(), torch.sin(pos[:, None] * f) * mag, rtol=0, atol=1e-6)
    if rot.get("scaling"):
        plain_f = rot["base"] ** (-2.0 * torch.arange(rot["dims"] // 2, dtype=torch.float64) / rot["dims"])
        assert not torch.allclose(f, plain_f)


def test_a_pairing_the_other_mixers_do_not_know_is_refused():
    from toyinfer_b200.parts import BuildContext, PartSpec, build_part
    ctx = BuildContext(dtype=torch.float32, device=torch.device("cpu"), hidden_size=32)
    ctx.positions["r"] = build_part("position", PartSpec("rotary_half", {"dim": 8, "theta": 1e4, "max_positions": 16, "pairing": "neighbours"}), ctx, "")
    with pytest.raises(ValueError, match="pairs neighbours"):
        build_part("mixer", PartSpec("gqa_attention", {"n_heads": 2, "n_kv_heads": 1, "head_dim": 8, "position": "r"}), ctx, "a.")
    with pytest.raises(ValueError, match="pairing"):
        build_part("position", PartSpec("rotary_half", {"dim": 8, "theta": 1e4, "max_positions": 16, "pairing": "thirds"}), ctx, "")


def test_the_cache_places_a_tuple_of_requests():
    """An entry that asks with (keys and values, a state) gets both, the keys in a group with other entries of the same
    shape, the state zeroed when its slot is handed out again."""
    from toyinfer_b200.cache import CacheManager, KVView, StateView, bytes_per_token
    from toyinfer_b200.parts import KVRequest, StateRequest
    kv, kv2 = KVRequest(2, 8, 0, True, 4), KVRequest(1, 16)
    reqs = [(kv, StateRequest((3, 5))), kv2, (kv, StateRequest((2,))), None, StateRequest((7,))]
    c = CacheManager(reqs, 256, 3, 128, torch.float32, "cpu")
    assert len(c.kv_groups) == 2
    a, b = c.view(0), c.view(2)
    assert isinstance(a, tuple) and isinstance(a[0], KVView) and isinstance(a[1], StateView) and isinstance(c.view(1), KVView)
    assert a[0].page_table is b[0].page_table and a[0].k_pages.data_ptr() != b[0].k_pages.data_ptr()
    assert tuple(a[0].v_pages.shape[1:]) == (2, 64, 4) and tuple(a[1].state.shape) == (4, 3, 5) and tuple(b[1].state.shape) == (4, 2)
    assert c.view(3) is None and tuple(c.view(4).state.shape) == (4, 7)
    assert bytes_per_token(reqs, torch.float32) == 4 * (2 * (8 + 4) * 2 + 2 * 16)
    s = c.allocate_slot()
    c.reserve(s, 100)
    a[1].state[s] = 3.0
    b[1].state[s] = 4.0
    c.release(s)
    s2 = c.allocate_slot()
    assert s2 == s and float(a[1].state[s].abs().sum()) == 0.0 and float(b[1].state[s].abs().sum()) == 0.0
