"""Bolisun's mechanisms one at a time against the plain implementation (tests/plain/bolisun_plain.py): streams without a
scale per channel, the clamped gated feed-forward, softmax attention under a window that keeps the first positions (biases,
per-head norms, neighbour-paired rotation with stretched frequencies), retention, the two side by side, the softmax router
with its correction and groups, and the experts.  Mixers run as prompts, single tokens, pieces of several sizes and unequal
batches, in slots and pages that another sequence used before; loud tokens (a row thirty times the others) stand among the
kept first positions, just behind them, at page borders and where windows end, so that every query that should or should
not see them shows."""
from __future__ import annotations

import math

import pytest
import torch

from plain import bolisun_plain as plain
from test_bagasun_parts_gpu import loud_inputs, short_names
from test_kadodra_parts_gpu import DEV, DT, bind_random, ctx_for, tol
from test_tusasun_parts_gpu import check_all_schedules, feed, inputs, schedules

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("S,H", [(1, 40), (3, 72), (4, 300)])
def test_streams_take_an_output_without_a_channel_scale(dtype, S, H):
    from toyinfer_b200.kernels import hyper
    g = torch.Generator().manual_seed(S * H)
    M, eps = 7, 1e-5
    X = torch.randn(M, S, H, generator=g) * 2
    y = (torch.randn(M, H, generator=g) * 3).to(dtype)
    c = {"in": torch.randn(S, generator=g), "out": torch.randn(S, generator=g), "mix": torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)}
    w = torch.rand(H, generator=g) + 0.5
    new = plain.connect(X.double(), y.double(), {k: v.double() for k, v in c.items()})
    Xd = X.reshape(M, S * H).to(DEV).clone()
    out = hyper.hyper_norm(Xd, hyper.StreamUpdate(y.to(DEV), None, c["mix"].to(DEV), c["out"].to(DEV)), c["in"].to(DEV), w.to(DEV), eps, dtype, S)
    torch.testing.assert_close(Xd.cpu().double().view(M, S, H), new, rtol=1e-5, atol=1e-5)
    want = plain.rms_norm(plain.read_streams(new, {k: v.double() for k, v in c.items()}), w, eps)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype, 2.0))


@pytest.mark.parametrize("dtype", DT)
def test_clamped_gate_both_layouts(dtype):
    """Values on both sides of the limit, of both signs: the gate is cut from above only, the up value on both sides."""
    import toyinfer_b200.kernels as K
    from toyinfer_b200.kernels import moe as KM
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(11, 2 * 37 + 3, generator=g) * 3).to(dtype)
    x = gu[:, :74].double()

    def want(gate, up, limit):
        gc, uc = torch.clamp(gate, max=limit), torch.clamp(up, min=-limit, max=limit)
        return gc * plain.sigmoid(1.702 * gc) * (uc + 1.0)
    for limit in (0.7, 2.0, 50.0):
        got = K.gated_act(gu.to(DEV)[:, :74], "clamped_swish", limit=limit).cpu().double()
        torch.testing.assert_close(got, want(x[:, :37], x[:, 37:], limit), **tol(dtype, 4.0))
        got = K.gated_act(gu.to(DEV)[:, :74], "clamped_swish", pairs=True, limit=limit).cpu().double()
        torch.testing.assert_close(got, want(x[:, 0::2], x[:, 1::2], limit), **tol(dtype, 4.0))
        dense = gu[:, :74].contiguous().to(DEV)
        torch.testing.assert_close(KM.act_pair(dense, limit, 1.702, 1.0).cpu().double(), want(x[:, :37], x[:, 37:], limit), **tol(dtype, 4.0))
    # no limit, no sharpening, no shift: silu(gate) * up
    torch.testing.assert_close(KM.act_pair(dense, float("inf"), 1.0, 0.0).cpu().double(), plain.silu(x[:, :37]) * x[:, 37:], **tol(dtype, 4.0))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hidden,ff,M,limit", [(56, 40, 5, 0.5), (64, 200, 130, 2.0), (40, 9, 1, 4.0), (128, 256, 70, 1.0)])
def test_clamped_gated_feed_forward(dtype, hidden, ff, M, limit):
    from toyinfer_b200.parts import PartSpec, build_part
    m = build_part("feed_forward", PartSpec("gated_dense", {"intermediate_size": ff, "act": "clamped_swish", "limit": limit}),
                   ctx_for(dtype, hidden), "f.")
    w = short_names(bind_random(m, 4, dtype, lambda cpu: [cpu[k].mul_(6.0) for k in ("f.gate", "f.up")]), "f.")
    x = inputs([M], hidden, 6, dtype)[0]
    got = m.forward(x.to(DEV), None).cpu().double()
    pre = x.double() @ w["gate"].T
    assert (pre > limit).any() and (pre < limit).any()         # the limit matters and is not everything
    torch.testing.assert_close(got, plain.clamped_ff(x.double(), w, limit), **tol(dtype, 4.0))


# ---------------------------------------------------------------------------
STRETCH = {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}
KEPT = [
    dict(n_heads=6, n_kv_heads=2, dim=16, vdim=24, window=40, keep_first=5, rot=dict(base=1e4, dims=8)),
    dict(n_heads=5, n_kv_heads=5, dim=8, vdim=8, window=1, keep_first=1),                   # itself and position 0
    dict(n_heads=4, n_kv_heads=1, dim=20, vdim=12, window=64, keep_first=3, rot=dict(base=300.0, dims=12, scaling=STRETCH)),   # exactly a page
    dict(n_heads=2, n_kv_heads=1, dim=128, vdim=64, window=65, keep_first=64, rot=dict(base=1e6, dims=128)),        # a page kept
    dict(n_heads=3, n_kv_heads=3, dim=40, vdim=200, window=130, keep_first=0, rot=dict(base=50.0, dims=2)),         # nothing kept
    dict(n_heads=8, n_kv_heads=2, dim=64, vdim=64, window=0, keep_first=7),                 # every earlier key: nothing to keep
    dict(n_heads=2, n_kv_heads=2, dim=12, vdim=36, window=9, keep_first=70),                # more kept than a window, past a page
    dict(n_heads=4, n_kv_heads=2, dim=64, vdim=128, window=200, keep_first=33, rot=dict(base=1e4, dims=64, scaling=dict(STRETCH, original=256))),
    dict(n_heads=4, n_kv_heads=1, dim=128, vdim=128, window=31, keep_first=2, rot=dict(base=1e4, dims=32)),
    # sizes that the tensor-core kernels take in bfloat16: kept positions that end inside a second tile; a window of a tile
    dict(n_heads=4, n_kv_heads=2, dim=128, vdim=128, window=70, keep_first=66),
    dict(n_heads=2, n_kv_heads=2, dim=64, vdim=64, window=64, keep_first=1, rot=dict(base=1e4, dims=64)),
]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("pairing", ["half", "neighbours"])
@pytest.mark.parametrize("H,G,dim,vdim,rot", [(3, 1, 48, 20, 12), (4, 2, 64, 128, 32), (2, 2, 128, 64, 128), (2, 1, 256, 256, 64), (5, 5, 128, 128, 0)])
def test_heads_prepared_one_by_one(dtype, pairing, H, G, dim, vdim, rot):
    """The kernel alone (a lane a run of elements for bfloat16 heads of 64, 128 and 256, a lane an element otherwise): biases,
    one norm weight for all heads, either pairing of the rotation, rows of a wider projection, keys and values in their pages."""
    from toyinfer_b200.cache import CacheManager
    from toyinfer_b200.kernels import attention_window as KW
    from toyinfer_b200.parts import KVRequest
    from toyinfer_b200.parts.rope import rotary_tables
    from test_kadodra_parts_gpu import batch_for
    g = torch.Generator().manual_seed(dim + rot)
    N = H * dim + G * (dim + vdim)
    lens, starts = [70, 3], [5, 64]
    M = sum(lens)
    y = (torch.randn(M, N + 16, generator=g) * 2).to(dtype)
    bias, qw, kw = torch.randn(N, generator=g), torch.rand(dim, generator=g) + 0.5, torch.rand(dim, generator=g) + 0.5
    tables = None
    if rot:
        cos, sin = rotary_tables(rot, 1e3, 256)
        tables = (cos.to(DEV), sin.to(DEV), rot)
    cache = CacheManager([KVRequest(G, dim, 0, True, vdim if vdim != dim else 0)], 64 * 8, 2, 256, dtype, DEV)
    slots = [cache.allocate_slot() for _ in lens]
    for s_, st, n in zip(slots, starts, lens):
        cache.reserve(s_, st + n)
    cache.flush()
    yd = y.to(DEV)
    KW.head_prepare(yd[:, :N], bias.to(DEV), qw.to(DEV), kw.to(DEV), 1e-5, tables, pairing, H, G, dim, vdim, cache.view(0),
                    batch_for("mixed", slots, starts, lens, cache.scratch_slot))
    x = y[:, :N].double() + bias.double()
    pos = torch.cat([torch.arange(st, st + n) for st, n in zip(starts, lens)])

    def heads(t, n, w):
        t = t.reshape(M, -1, n)
        t = t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-5) * w.double()
        if rot:
            c, s_ = cos.double()[pos][:, None, :], sin.double()[pos][:, None, :]
            a, b = (t[..., 0:rot:2], t[..., 1:rot:2]) if pairing == "neighbours" else (t[..., :rot // 2], t[..., rot // 2:rot])
            ra, rb = a * c - b * s_, b * c + a * s_
            t = t.clone()
            if pairing == "neighbours":
                t[..., 0:rot:2], t[..., 1:rot:2] = ra, rb
            else:
                t[..., :rot // 2], t[..., rot // 2:rot] = ra, rb
        return t.reshape(M, -1)
    want = torch.cat([heads(x[:, :H * dim], dim, qw), heads(x[:, H * dim:(H + G) * dim], dim, kw), x[:, (H + G) * dim:]], dim=1)
    torch.testing.assert_close(yd[:, :N].cpu().double(), want, **tol(dtype, 4.0))
    assert torch.equal(yd[:, N:].cpu(), y[:, N:])                    # the columns after q, k, v are left alone
    view = cache.view(0)
    table = view.page_table.cpu()
    o = 0
    for s_, st, n in zip(slots, starts, lens):
        for i in (0, n - 1):
            p = st + i
            page = int(table[s_, p // 64])
            krow = view.k_pages[page, :, p % 64].reshape(-1).cpu()
            vrow = view.v_pages[page, :, p % 64].reshape(-1).cpu()
            assert torch.equal(krow, yd[o + i, H * dim:(H + G) * dim].cpu()) and torch.equal(vrow, yd[o + i, (H + G) * dim:N].cpu())
        o += n


def make_kept(dtype, c, hidden=56, seed=3, **options):
    from toyinfer_b200.parts import PartSpec, build_part
    c = dict(c)
    rot = c.pop("rot", None)
    positions, position = {}, None
    if rot:
        position = "r"
        positions["r"] = build_part("position", PartSpec("rotary_half", {"dim": rot["dims"], "theta": rot["base"], "max_positions": 2048,
                                                                         "scaling": rot.get("scaling"), "pairing": "neighbours"}),
                                    ctx_for(dtype, hidden), "")
    m = build_part("mixer", PartSpec("kept_window_attention", dict(c, scale=0.35, eps=1e-5, position=position, **options)),
                   ctx_for(dtype, hidden, positions), "a.")
    w = bind_random(m, seed, dtype)
    mcfg = {"heads": c["n_heads"], "kv_heads": c["n_kv_heads"], "dim": c["dim"], "vdim": c["vdim"], "scale": 0.35}
    if c["window"]:
        mcfg["mask"] = {"size": c["window"], "keep_first": c["keep_first"]}
    if rot:
        mcfg["rot"] = rot
    return m, short_names(w), mcfg


def test_which_kernels_take_the_kept_window(monkeypatch):
    """bfloat16 heads of 64 or 128 run prompts, pieces and single tokens on the tensor-core kernels, kept positions and
    all; the CUDA-core kernels give the same within the rounding of the weights."""
    from toyinfer_b200.kernels import attention_window as KW
    dtype = torch.bfloat16
    m, w, mcfg = make_kept(dtype, KEPT[-2])
    xs = [loud_inputs(n, 56, 5 + n, [j for j in (0, 65, 66, 130) if j < n]).to(dtype) for n in (330, 67)]
    calls = []
    real = KW._fn

    def spy(name, sig):
        calls.append(name)
        return real(name, sig)
    monkeypatch.setattr(KW, "_fn", spy)
    sch = schedules([330, 67])
    got = {name: feed(m, m.memory_request(), xs, s_, dtype) for name, s_ in sch.items()}
    assert "ti_attn_window_tc" in calls and "ti_attn_decode_mma_scored" in calls
    assert "ti_attn_window" not in calls and "ti_attn_window_decode" not in calls
    monkeypatch.setattr(KW, "tensor_cores", False)
    calls.clear()
    other = {name: feed(m, m.memory_request(), xs, s_, dtype) for name, s_ in sch.items()}
    assert "ti_attn_window" in calls and "ti_attn_window_decode" in calls and "ti_attn_window_tc" not in calls
    wants = [plain.window_attention(x.double(), w, mcfg, 1e-5) for x in xs]
    for name in sch:
        for g, o, want in zip(got[name], other[name], wants):
            torch.testing.assert_close(g, want, **tol(dtype, 30.0), msg=lambda e: f"{name}, tensor cores: {e}")
            torch.testing.assert_close(o, want, **tol(dtype, 30.0), msg=lambda e: f"{name}, CUDA cores: {e}")


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", KEPT)
def test_kept_window_attention_every_way_of_feeding(dtype, c):
    """Loud rows at the first tokens, at the last kept position and the one behind it, at both sides of two page borders,
    and where the longest sequence's late windows end."""
    m, w, mcfg = make_kept(dtype, c)
    lens = [300, 129, 3]
    k = c["keep_first"]
    loud = sorted({0, 2, 63, 64, 127, 128, 250, max(k - 1, 0), k, 299 - c["window"], 300 - c["window"]})
    xs = [loud_inputs(n, 56, 5 + i, [j for j in loud if 0 <= j < n]).to(dtype) for i, n in enumerate(lens)]
    wants = [plain.window_attention(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype, scale=30.0)


@pytest.mark.parametrize("dtype", DT)
def test_kept_window_attention_without_its_options(dtype):
    c = dict(n_heads=4, n_kv_heads=2, dim=16, vdim=16, window=50, keep_first=4)
    m, w, mcfg = make_kept(dtype, c, biases=False, head_norm=False)
    assert set(w) == {"q", "k", "v", "o"}
    w.update({"q.b": torch.zeros(64), "k.b": torch.zeros(32), "v.b": torch.zeros(32), "o.b": torch.zeros(56),
              "q.norm": None, "k.norm": None})
    xs = inputs([150, 20], 56, 8, dtype)

    def unnormed(x):
        # the plain function norms; without weights the heads pass as they are, so the norm is undone by hand
        T = x.shape[0]
        q = (x @ w["q"].T).view(T, 4, 16)
        k = (x @ w["k"].T).view(T, 2, 16)
        v = (x @ w["v"].T).view(T, 2, 16)
        o = torch.zeros(T, 4, 16, dtype=torch.float64)
        for h in range(4):
            for i in range(T):
                js = [j for j in range(i + 1) if plain.visible(i, j, mcfg["mask"])]
                s = (k[js, h // 2] @ q[i, h]) * 0.35
                p = torch.exp(s - s.max())
                o[i, h] = (p / p.sum()) @ v[js, h // 2]
        return o.reshape(T, 64) @ w["o"].T
    check_all_schedules(m, xs, [unnormed(x.double()) for x in xs], dtype, scale=10.0)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("far", [0, 4, 5])
def test_one_kept_key_among_hundreds(dtype, far):
    """The queries' and keys' norm weights are ten times the usual and the token at ``far`` carries a value like no other:
    with five kept positions, late queries find position 0 and 4 however far back they are, and never position 5."""
    c = dict(n_heads=2, n_kv_heads=1, dim=32, vdim=16, window=24, keep_first=5)
    m, w, mcfg = make_kept(dtype, c, seed=9)
    T = 500
    x = loud_inputs(T, 56, 31, [far], factor=40.0).to(dtype)
    want = plain.window_attention(x.double(), w, mcfg, 1e-5)
    quiet = x.clone()
    quiet[far] /= 40.0
    base = plain.window_attention(quiet.double(), w, mcfg, 1e-5)
    seen = (want[100:] - base[100:]).abs().amax() > 1e-3
    assert bool(seen) == (far < 5)
    check_all_schedules(m, [x], [want], dtype, scale=40.0)


# ---------------------------------------------------------------------------
RETENTION = [dict(n_heads=3, dim=12, vdim=20, decay=[0.9, 0.97, 0.995]), dict(n_heads=1, dim=40, vdim=40, decay=[0.96]),
             dict(n_heads=4, dim=8, vdim=16, decay=[0.5, 0.9, 0.99, 1.0]), dict(n_heads=2, dim=128, vdim=64, decay=[0.97, 0.999]),
             dict(n_heads=2, dim=64, vdim=128, decay=[0.9, 0.95])]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("chunked_from", [None, 2])
@pytest.mark.parametrize("c", RETENTION)
def test_retention_every_way_of_feeding(dtype, c, chunked_from, monkeypatch):
    """``chunked_from``: every step that brings a sequence two tokens or more runs the chunked form of the recurrence."""
    from toyinfer_b200.kernels import lightning as KS
    from toyinfer_b200.parts import PartSpec, build_part
    if chunked_from is not None:
        monkeypatch.setattr(KS, "CHUNKED_FROM", chunked_from)
    m = build_part("mixer", PartSpec("retention", dict(c, eps=1e-5)), ctx_for(dtype, 56), "a.")
    w = short_names(bind_random(m, 3, dtype))
    xs = inputs([300, 129, 3], 56, 5, dtype)
    mcfg = {"heads": c["n_heads"], "dim": c["dim"], "vdim": c["vdim"], "decay": c["decay"]}
    wants = [plain.retention(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype)


@pytest.mark.parametrize("dtype", DT)
def test_retention_over_many_single_tokens(dtype):
    from toyinfer_b200.parts import PartSpec, build_part
    c = dict(n_heads=2, dim=16, vdim=24, decay=[0.999, 0.9])
    m = build_part("mixer", PartSpec("retention", dict(c, eps=1e-6)), ctx_for(dtype, 40), "a.")
    w = short_names(bind_random(m, 13, dtype))
    x = inputs([400], 40, 15, dtype)[0]
    want = plain.retention(x.double(), w, {"heads": 2, "dim": 16, "vdim": 24, "decay": c["decay"]}, 1e-6)
    got = feed(m, m.memory_request(), [x], [[(0, 5)]] + [[(0, 1)]] * 395, dtype)
    torch.testing.assert_close(got[0], want, **tol(dtype, 3.0))


# ---------------------------------------------------------------------------
def make_pair(dtype, left, right, ls, rs, hidden=56, seed=5):
    from toyinfer_b200.parts import PartSpec, build_part
    left = dict(left)
    rot = left.pop("rot", None)
    positions, position = {}, None
    if rot:
        position = "r"
        positions["r"] = build_part("position", PartSpec("rotary_half", {"dim": rot["dims"], "theta": rot["base"], "max_positions": 2048,
                                                                         "scaling": rot.get("scaling"), "pairing": "neighbours"}),
                                    ctx_for(dtype, hidden), "")
    spec = PartSpec("side_by_side", {
        "left": PartSpec("kept_window_attention", dict(left, scale=0.3, eps=1e-5, position=position)),
        "right": PartSpec("retention", dict(right, eps=1e-5)), "left_scale": ls, "right_scale": rs})
    m = build_part("mixer", spec, ctx_for(dtype, hidden, positions), "a.")
    w = short_names(bind_random(m, seed, dtype))
    mcfg = {"left": {"heads": left["n_heads"], "kv_heads": left["n_kv_heads"], "dim": left["dim"], "vdim": left["vdim"], "scale": 0.3,
                     "mask": {"size": left["window"], "keep_first": left["keep_first"]}},
            "right": {"heads": right["n_heads"], "dim": right["dim"], "vdim": right["vdim"], "decay": right["decay"]},
            "left_scale": ls, "right_scale": rs}
    if rot:
        mcfg["left"]["rot"] = rot
    return m, w, mcfg


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("left,right,ls,rs", [
    (KEPT[0], RETENTION[0], 0.7, 1.3),             # the attention's rows are no multiple of eight: the state mixer's are moved up
    (KEPT[2], RETENTION[1], 1.0, 1.0),
    (KEPT[7], RETENTION[3], 0.25, 2.0),
    (KEPT[6], RETENTION[2], 1.5, 0.0),             # a side that is switched off
])
def test_two_mixers_side_by_side(dtype, left, right, ls, rs):
    m, w, mcfg = make_pair(dtype, left, right, ls, rs)
    assert m.joined
    xs = [loud_inputs(n, 56, 5 + i, [j for j in (0, 2, 63, 64, 127, 128, 250) if j < n]).to(dtype) for i, n in enumerate([300, 129, 3])]
    wants = [plain.parallel_mixer(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype, scale=30.0)


@pytest.mark.parametrize("dtype", DT)
def test_side_by_side_members_that_run_whole(dtype):
    """A member that cannot hand out its projections' rows (lightning attention) runs whole beside the other: two states."""
    from toyinfer_b200.parts import PartSpec, build_part
    a = PartSpec("lightning", dict(n_heads=2, dim=16, vdim=8, decay=[0.9, 0.99], eps=1e-5))
    b = PartSpec("retention", dict(n_heads=3, dim=8, vdim=12, decay=[0.8, 0.95, 0.99], eps=1e-5))
    m = build_part("mixer", PartSpec("side_by_side", {"left": a, "right": b, "left_scale": 0.6, "right_scale": -1.2}), ctx_for(dtype, 40), "a.")
    assert not m.joined
    bind_random(m, 21, dtype)
    xs = inputs([90, 7], 40, 22, dtype)
    alone = []
    for part, pre in ((m.left, 0), (m.right, 1)):
        alone.append(feed(part, part.memory_request(), xs, schedules([90, 7])["whole"], dtype))
    wants = [0.6 * l - 1.2 * r for l, r in zip(*alone)]
    check_all_schedules(m, xs, wants, dtype)


# ---------------------------------------------------------------------------
def test_router_choices_against_the_rule():
    """Logits and corrections made so that the cases of the rule all occur: a correction that changes the choice but not
    the weights; negative choice scores, where an expert outside the kept groups must not win although its score counts
    as less than nothing; equal scores (the lower index wins); all groups kept; no groups."""
    from toyinfer_b200.kernels import moe as KM
    g = torch.Generator().manual_seed(4)
    for E, top, groups, keep, scale in [(6, 2, 3, 2, 1.5), (8, 4, 4, 2, 0.5), (16, 3, 4, 3, 2.0), (5, 3, 0, 0, 1.0), (4, 1, 2, 2, 1.0),
                                        (12, 2, 6, 1, 3.0)]:
        M = 64
        z = torch.randn(M, E + 3, generator=g) * 2
        z[5] = 0.0                                       # all equal
        z[6, :E] = torch.tensor([1.0, 1.0] * (E // 2) + [1.0] * (E % 2))
        corr = torch.randn(E, generator=g) * 0.3 - 1.0   # every choice score is negative
        r = {"experts": E, "top": top, "scale": scale}
        if groups:
            r["groups"] = {"count": groups, "keep": keep}
        perm, off, weight = KM.route_softmax(z.to(DEV)[:, :E], corr.to(DEV), E, top, groups, keep, scale)
        perm, off, weight = perm.cpu(), off.cpu(), weight.cpu()
        expert_of = torch.empty(M * top, dtype=torch.long)
        for e in range(E):
            expert_of[perm[off[e]:off[e + 1]].long()] = e
        assert off[0] == 0 and off[E] == M * top and sorted(perm.tolist()) == list(range(M * top))
        for m in range(M):
            chosen, w = plain.route(z[m, :E], corr, r)
            assert expert_of[m * top:(m + 1) * top].tolist() == chosen, (E, top, groups, keep, m)
            torch.testing.assert_close(weight[m * top:(m + 1) * top].double(), w, rtol=1e-5, atol=1e-6)
        # without a correction
        perm, off, weight = KM.route_softmax(z.to(DEV)[:, :E], None, E, top, groups, keep, scale)
        expert_of = torch.empty(M * top, dtype=torch.long)
        for e in range(E):
            expert_of[perm.cpu()[off[e]:off[e + 1]].long()] = e
        for m in (0, 5, 6, 63):
            assert expert_of[m * top:(m + 1) * top].tolist() == plain.route(z[m, :E], torch.zeros(E), r)[0]


MOE = [dict(n_experts=6, top=2, intermediate_size=24, n_groups=3, keep=2, scale=1.5, shared_size=16),
       dict(n_experts=5, top=3, intermediate_size=16),
       dict(n_experts=4, top=1, intermediate_size=32, n_groups=2, keep=2, shared_size=24),
       dict(n_experts=8, top=4, intermediate_size=8, n_groups=4, keep=2, scale=0.5)]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M", [1, 7, 700])           # single tokens, a few, and enough pairs per expert for the padded tensor-core groups
@pytest.mark.parametrize("c", MOE)
def test_experts_under_the_softmax_router(dtype, c, M):
    from toyinfer_b200.parts import PartSpec, build_part
    hidden = 64
    m = build_part("feed_forward", PartSpec("softmax_moe", dict(c)), ctx_for(dtype, hidden), "f.")
    w = short_names(bind_random(m, 8, dtype, lambda cpu: cpu["f.router"].mul_(3.0)), "f.")
    x = inputs([M], hidden, 10 + M, dtype)[0]
    f = {"router": {"experts": c["n_experts"], "top": c["top"], "scale": c.get("scale", 1.0)}}
    if c.get("n_groups"):
        f["router"]["groups"] = {"count": c["n_groups"], "keep": c["keep"]}
    if c.get("shared_size"):
        f["shared"] = {"ff": c["shared_size"]}
    got = m.forward(x.to(DEV), None).cpu().double()
    want = plain.experts_ff(x.double(), w, f)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, **tol(dtype, 2.0))
    else:           # a close call of the router may fall the other way for a token: all but a few rows agree
        bad = ((got - want).abs() > 3e-2 * want.abs() + 4e-2).any(dim=1)
        assert int(bad.sum()) <= max(1, M // 50), f"{int(bad.sum())} of {M} rows differ"
