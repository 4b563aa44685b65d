"""Bagasun's mechanisms one at a time against the plain implementation (tests/plain/bagasun_plain.py): the float32 stream
with normed sublayer outputs, the gelu-gated feed-forward, attention with sigmoid weights and a logarithmic distance term,
differential attention with rotated maps, and the Mamba-2 recurrence with its gated group norm.  Mixers run as prompts,
single tokens, pieces of several sizes and unequal batches, in slots and pages that another sequence used before; loud
tokens (a row thirty times the others) stand at page borders so that every query that should or should not see them shows."""
from __future__ import annotations

import pytest
import torch

from plain import bagasun_plain as plain
from test_kadodra_parts_gpu import DEV, DT, bind_random, ctx_for, tol
from test_tusasun_parts_gpu import check_all_schedules, feed, inputs

pytestmark = pytest.mark.gpu


def loud_inputs(T, hidden, seed, loud=(), factor=30.0):
    """Random rows; the rows at ``loud`` are ``factor`` times larger."""
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(seed))
    for j in loud:
        x[j] *= factor
    return x


def short_names(cpu, prefix="a."):
    return {k[len(prefix):]: v.double() for k, v in cpu.items() if k.startswith(prefix)}


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H,scalar", [(40, True), (300, True), (72, False), (1100, True)])
def test_stream_takes_a_normed_output_and_is_normed_again(dtype, H, scalar):
    from toyinfer_b200.kernels import wide
    g = torch.Generator().manual_seed(H)
    M, eps = 9, 1e-5
    h = torch.randn(M, H, generator=g) * 3
    y = (torch.randn(M, H, generator=g) * 5).to(dtype)
    wp = torch.tensor([0.7]) if scalar else torch.rand(H, generator=g) + 0.5
    wn = torch.tensor([1.3]) if scalar else torch.rand(H, generator=g) + 0.5
    new = h.double() + plain.unit_rms(y.double(), eps) * wp.double()
    hd = h.to(DEV).clone()
    out = wide.post_norm_add_norm(hd, wide.PostNormed(y.to(DEV), wp.to(DEV), eps), wn.to(DEV), eps, dtype)
    torch.testing.assert_close(hd.cpu().double(), new, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.cpu().double(), plain.unit_rms(new, eps) * wn.double(), **tol(dtype, 2.0))
    # nothing pending: the stream stays as it is
    hd = h.to(DEV).clone()
    out = wide.post_norm_add_norm(hd, None, wn.to(DEV), eps, dtype)
    assert torch.equal(hd.cpu(), h)
    torch.testing.assert_close(out.cpu().double(), plain.unit_rms(h.double(), eps) * wn.double(), **tol(dtype, 2.0))
    # gathered rows with something pending: the stream is left alone
    rows = torch.tensor([5, 0, 5, 8], dtype=torch.int32, device=DEV)
    out = wide.post_norm_add_norm(hd, wide.PostNormed(y.to(DEV), wp.to(DEV), eps), wn.to(DEV), eps, dtype, rows=rows)
    assert torch.equal(hd.cpu(), h)
    torch.testing.assert_close(out.cpu().double(), (plain.unit_rms(new, eps) * wn.double())[[5, 0, 5, 8]], **tol(dtype, 2.0))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_activation_both_layouts(dtype, act):
    import toyinfer_b200.kernels as K
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(11, 2 * 37 + 3, generator=g) * 3).to(dtype)
    f = plain.gelu_tanh if act == "gelu_tanh" else plain.silu
    x = gu[:, :74].double()
    got = K.gated_act(gu.to(DEV)[:, :74], act).cpu().double()                 # rows of a wider matrix
    torch.testing.assert_close(got, f(x[:, :37]) * x[:, 37:], **tol(dtype, 4.0))
    got = K.gated_act(gu.to(DEV)[:, :74], act, pairs=True).cpu().double()
    torch.testing.assert_close(got, f(x[:, 0::2]) * x[:, 1::2], **tol(dtype, 4.0))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hidden,ff,M", [(56, 40, 5), (64, 200, 130), (40, 9, 1)])
def test_gelu_gated_feed_forward(dtype, hidden, ff, M):
    from toyinfer_b200.parts import PartSpec, build_part
    m = build_part("feed_forward", PartSpec("gated_dense", {"intermediate_size": ff, "act": "gelu_tanh"}), ctx_for(dtype, hidden), "f.")
    w = short_names(bind_random(m, 4, dtype), "f.")
    x = inputs([M], hidden, 6, dtype)[0]
    got = m.forward(x.to(DEV), None).cpu().double()
    torch.testing.assert_close(got, plain.gated_gelu_ff(x.double(), w["gate"], w["up"], w["down"]), **tol(dtype, 2.0))


# ---------------------------------------------------------------------------
SIGMOID = [
    dict(n_heads=6, n_kv_heads=2, dim=16, vdim=24, window=40),
    dict(n_heads=5, n_kv_heads=5, dim=8, vdim=8, window=1),                  # every query sees itself only
    dict(n_heads=4, n_kv_heads=1, dim=20, vdim=12, window=64),               # exactly a page
    dict(n_heads=2, n_kv_heads=1, dim=128, vdim=64, window=65),
    dict(n_heads=3, n_kv_heads=3, dim=40, vdim=200, window=130),
    dict(n_heads=8, n_kv_heads=2, dim=64, vdim=64, window=0),                # every earlier key
    dict(n_heads=2, n_kv_heads=2, dim=12, vdim=36, window=1000),             # longer than any sequence here
    # sizes that the tensor-core kernel takes in bfloat16: windows inside a tile, of three pages and a bit, of one key
    dict(n_heads=4, n_kv_heads=2, dim=64, vdim=128, window=200),
    dict(n_heads=2, n_kv_heads=1, dim=128, vdim=128, window=31),
    dict(n_heads=3, n_kv_heads=3, dim=64, vdim=64, window=1),
]


def make_sigmoid(dtype, c, hidden=56, seed=3, **options):
    from toyinfer_b200.parts import PartSpec, build_part
    m = build_part("mixer", PartSpec("sigmoid_attention", dict(c, scale=0.35, eps=1e-5, **options)), ctx_for(dtype, hidden), "a.")

    def edit(cpu):
        H = c["n_heads"]
        if "a.r1" in cpu:           # heads that forget far keys, one that prefers them, one without a distance term
            cpu["a.r1"].copy_(torch.linspace(1.5, -0.4, H))
            cpu["a.r2"].copy_(torch.linspace(0.05, 2.0, H))
            cpu["a.r1"][H // 2] = 0.0
        if "a.pb" in cpu:
            cpu["a.pb"].copy_(torch.linspace(-3.0, 0.5, H))
    w = bind_random(m, seed, dtype, edit)
    mcfg = {"heads": c["n_heads"], "kv_heads": c["n_kv_heads"], "dim": c["dim"], "vdim": c["vdim"], "scale": 0.35}
    if c["window"]:
        mcfg["mask"] = {"size": c["window"]}
    return m, short_names(w), mcfg


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", SIGMOID)
def test_sigmoid_attention_every_way_of_feeding(dtype, c):
    """Loud rows at the first tokens, at both sides of two page borders and late in the longest sequence: their values
    are thirty times the others', so every query whose window holds one (and none whose window has just lost it) shows it."""
    m, w, mcfg = make_sigmoid(dtype, c)
    lens = [300, 129, 3]
    xs = [loud_inputs(n, 56, 5 + i, [j for j in (0, 2, 63, 64, 127, 128, 250) if j < n]).to(dtype) for i, n in enumerate(lens)]
    wants = [plain.sigmoid_attention(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype, scale=30.0)


@pytest.mark.parametrize("dtype", DT)
def test_sigmoid_attention_without_its_options(dtype):
    c = dict(n_heads=4, n_kv_heads=2, dim=16, vdim=16, window=50)
    m, w, mcfg = make_sigmoid(dtype, c, biases=False, row_norm=False, distance=False, head_bias=False)
    assert set(w) == {"q", "k", "v", "o"}
    xs = inputs([150, 20], 56, 8, dtype)
    wants = [plain.sigmoid_attention(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype, scale=10.0)


# ---------------------------------------------------------------------------
DIFF = [
    dict(n_heads=2, n_kv_heads=1, dim=24, vdim=40, window=33, rot=24, scaling=None, diff=0.3),            # the whole map rotated
    dict(n_heads=3, n_kv_heads=3, dim=32, vdim=16, window=100, rot=8, diff=0.8,
         scaling={"factor": 4.0, "low": 2.0, "high": 8.0, "original": 64}),
    dict(n_heads=6, n_kv_heads=2, dim=12, vdim=20, window=64, rot=0, scaling=None, diff=0.5),              # no rotation
    dict(n_heads=4, n_kv_heads=2, dim=64, vdim=128, window=65, rot=32, diff=0.2,
         scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}),
    dict(n_heads=4, n_kv_heads=1, dim=128, vdim=64, window=0, rot=64, scaling=None, diff=0.1),
    dict(n_heads=1, n_kv_heads=1, dim=16, vdim=8, window=1, rot=4, scaling=None, diff=0.6),
    dict(n_heads=2, n_kv_heads=2, dim=64, vdim=64, window=129, rot=64, scaling=None, diff=0.4),
    dict(n_heads=6, n_kv_heads=2, dim=128, vdim=128, window=200, rot=16, scaling=None, diff=0.7),
]


def make_diff(dtype, c, hidden=56, seed=3, gate=True):
    from toyinfer_b200.parts import PartSpec, build_part
    ctx = ctx_for(dtype, hidden)
    position = None
    if c["rot"]:
        position = "r"
        ctx.positions["r"] = build_part("position", PartSpec("rotary_half", {
            "dim": c["rot"], "theta": 3e3, "max_positions": 512, "scaling": dict(c["scaling"], kind="bands") if c["scaling"] else None}), ctx, "")
    m = build_part("mixer", PartSpec("diff_attention", dict(
        n_heads=c["n_heads"], n_kv_heads=c["n_kv_heads"], dim=c["dim"], vdim=c["vdim"], scale=0.3, window=c["window"], eps=1e-5,
        diff=c["diff"], position=position, gate=gate)), ctx, "a.")

    def edit(cpu):                   # a lambda well away from its constant part: e^1.2 - e^-0.8 + diff
        r = c["dim"] ** -0.5
        cpu["a.lq1"].fill_(1.2 * r), cpu["a.lk1"].fill_(r), cpu["a.lq2"].fill_(-0.8 * r), cpu["a.lk2"].fill_(r)
    w = bind_random(m, seed, dtype, edit)
    mcfg = {"heads": c["n_heads"], "kv_heads": c["n_kv_heads"], "dim": c["dim"], "vdim": c["vdim"], "scale": 0.3, "diff": c["diff"]}
    if c["window"]:
        mcfg["mask"] = {"size": c["window"]}
    if c["rot"]:
        mcfg["rot"] = {"base": 3e3, "dims": c["rot"], "scaling": c["scaling"]}
    return m, short_names(w), mcfg


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", DIFF)
def test_differential_attention_every_way_of_feeding(dtype, c):
    """Loud rows have keys thirty times the others' (six times in bfloat16, where the rounding of two such keys that stand
    side by side would otherwise decide between them): a query that sees one gives it most of a map's weight, one way or
    the other, and a query whose window has just lost it does not."""
    m, w, mcfg = make_diff(dtype, c)
    factor = 30.0 if dtype == torch.float32 else 6.0
    assert abs(m.lam - (c["diff"] + 3.3201 - 0.4493)) < 0.05
    lens = [300, 129, 3]
    xs = [loud_inputs(n, 56, 15 + i, [j for j in (0, 2, 63, 64, 127, 128, 250) if j < n], factor).to(dtype) for i, n in enumerate(lens)]
    wants = [plain.diff_attention(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype, scale=3.0)


@pytest.mark.parametrize("kind,c", [("sigmoid", SIGMOID[3]), ("sigmoid", SIGMOID[7]), ("sigmoid", SIGMOID[8]), ("sigmoid", SIGMOID[9]),
                                    ("diff", DIFF[3]), ("diff", DIFF[4]), ("diff", DIFF[6]), ("diff", DIFF[7])])
def test_tensor_core_prompts_and_pieces_agree_with_the_cuda_core_kernel(kind, c, monkeypatch):
    """bfloat16, keys and values of 64 or 128 elements: the same mixer through the tcgen05 kernel and through the CUDA-core
    kernel, on whole prompts and on pieces that begin in the middle of a page.  The two differ by the rounding of the
    weights to bfloat16 for the second product, and a masked key must not leak: a loud row stands just outside a window."""
    from toyinfer_b200.kernels import attention_window as KW
    from test_tusasun_parts_gpu import schedules
    dtype = torch.bfloat16
    m, w, mcfg = (make_sigmoid if kind == "sigmoid" else make_diff)(dtype, c)
    calls = []
    real = KW._fn

    def spy(name, sig):
        calls.append(name)
        return real(name, sig)
    monkeypatch.setattr(KW, "_fn", spy)
    lens = [333, 130, 64, 2]
    xs = [loud_inputs(n, 56, 40 + i, [j for j in (1, 63, 64, 140, 330) if j < n], 6.0).to(dtype) for i, n in enumerate(lens)]
    sch = schedules(lens)
    got = {name: feed(m, m.memory_request(), xs, s, dtype) for name, s in sch.items()}
    assert "ti_attn_window_tc" in calls and "ti_attn_window" not in calls
    monkeypatch.setattr(KW, "tensor_cores", False)
    calls.clear()
    for name, s in sch.items():
        want = feed(m, m.memory_request(), xs, s, dtype)
        for i, (g, x) in enumerate(zip(got[name], want)):
            # (the mixer's output is a sum over hundreds of bfloat16 values of size ten: a few hundredths either way)
            torch.testing.assert_close(g, x, rtol=3e-2, atol=0.15, msg=lambda e: f"{kind} {name}, sequence {i}: {e}")
    assert "ti_attn_window_tc" not in calls


@pytest.mark.parametrize("kind,c", [
    ("sigmoid", dict(n_heads=8, n_kv_heads=2, dim=64, vdim=64, window=0)),                    # every earlier key
    ("sigmoid", dict(n_heads=20, n_kv_heads=1, dim=128, vdim=128, window=150)),               # more heads than one block's sixteen rows
    ("sigmoid", dict(n_heads=3, n_kv_heads=3, dim=64, vdim=64, window=1)),
    ("diff", dict(n_heads=10, n_kv_heads=1, dim=64, vdim=128, window=300, rot=32, diff=0.2,
                  scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256})),       # twenty score maps on one kv head
    ("diff", dict(n_heads=2, n_kv_heads=2, dim=32, vdim=64, window=0, rot=0, scaling=None, diff=0.5)),
    ("diff", dict(n_heads=4, n_kv_heads=2, dim=64, vdim=128, window=65, rot=64, scaling=None, diff=0.7)),
])
def test_single_tokens_on_the_tensor_core_kernel(kind, c, monkeypatch):
    """bfloat16 and a key row as long as a value row (64 or 128 elements): single tokens run on the dense model's
    tensor-core kernel under this design's score rules (sigmoid weights with the distance term; two maps that share a key
    row, float32 results).  Two sequences of unequal length go on token by token from 450 and 75 positions, far enough for
    the longer one's keys to be split over blocks and merged where the window shows that many; loud rows stand where the
    windows end and at page borders.  The
    result is held against the plain implementation and against the CUDA-core kernel."""
    from toyinfer_b200.kernels import attention_window as KW
    dtype = torch.bfloat16
    m, w, mcfg = (make_sigmoid if kind == "sigmoid" else make_diff)(dtype, c)
    calls = []
    real = KW._fn

    def spy(name, sig):
        calls.append(name)
        return real(name, sig)
    monkeypatch.setattr(KW, "_fn", spy)
    lens, steps = [500, 125], 50
    loud = [0, 63, 64, 150, 151, 200, 201, 300, 301, 349, 350, 385, 386, 448, 460]
    xs = [loud_inputs(n, 56, 60 + i, [j for j in loud if j < n], 6.0).to(dtype) for i, n in enumerate(lens)]
    fn = plain.sigmoid_attention if kind == "sigmoid" else plain.diff_attention
    wants = [fn(x.double(), w, mcfg, 1e-5) for x in xs]
    sched = [[(0, lens[0] - steps), (1, lens[1] - steps)]] + [[(0, 1), (1, 1)] for _ in range(steps)]
    got = feed(m, m.memory_request(), xs, sched, dtype)
    assert "ti_attn_decode_mma_scored" in calls and "ti_attn_window_decode" not in calls
    assert ("ti_attn_window_merge" in calls) == (c["window"] in (0, 300))
    for g, want in zip(got, wants):
        torch.testing.assert_close(g[-steps:], want[-steps:], **tol(dtype, 30.0 if kind == "sigmoid" else 3.0))
    monkeypatch.setattr(KW, "tensor_cores", False)
    calls.clear()
    slow = feed(m, m.memory_request(), xs, sched, dtype)
    assert "ti_attn_window_decode" in calls and "ti_attn_decode_mma_scored" not in calls
    for i, (g, x) in enumerate(zip(got, slow)):
        torch.testing.assert_close(g[-steps:], x[-steps:], rtol=3e-2, atol=0.15, msg=lambda e: f"{kind}, sequence {i}: {e}")


@pytest.mark.parametrize("dtype", DT)
def test_differential_attention_without_a_gate(dtype):
    c = DIFF[0]
    m, w, mcfg = make_diff(dtype, c, gate=False)
    assert "g" not in w
    xs = inputs([90, 5], 56, 3, dtype)
    wants = [plain.diff_attention(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype, scale=3.0)


# ---------------------------------------------------------------------------
SSM = [
    dict(n_heads=4, vdim=8, state=16, groups=2, conv=4, norm_groups=2),
    dict(n_heads=3, vdim=20, state=44, groups=1, conv=2, norm_groups=1),          # a state that is no multiple of eight
    dict(n_heads=2, vdim=64, state=128, groups=2, conv=4, norm_groups=4),
    dict(n_heads=6, vdim=16, state=8, groups=6, conv=1, norm_groups=3),           # a group per head, no convolution to speak of
    dict(n_heads=2, vdim=5, state=200, groups=1, conv=7, norm_groups=2),
]


def make_ssm(dtype, c, hidden=56, seed=3):
    from toyinfer_b200.parts import PartSpec, build_part
    m = build_part("mixer", PartSpec("mamba2", dict(c, eps=1e-5)), ctx_for(dtype, hidden), "a.")

    def edit(cpu):                  # decays from nearly none to nearly all, so that a lost or doubled state shows
        H = c["n_heads"]
        cpu["a.A_log"].copy_(torch.linspace(-5.0, 1.5, H))
        cpu["a.dt_bias"].copy_(torch.linspace(-3.0, 1.0, H))
    w = bind_random(m, seed, dtype, edit)
    mcfg = {"heads": c["n_heads"], "vdim": c["vdim"], "state": c["state"], "groups": c["groups"], "conv": c["conv"],
            "norm_groups": c["norm_groups"]}
    return m, short_names(w), mcfg


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", SSM)
def test_mamba2_every_way_of_feeding(dtype, c):
    m, w, mcfg = make_ssm(dtype, c)
    xs = inputs([300, 129, 3], 56, 5, dtype)
    wants = [plain.mamba2(x.double(), w, mcfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c,segment", [(SSM[0], 16), (SSM[1], 16), (SSM[2], 32), (SSM[4], 48), (SSM[2], None)])
def test_mamba2_segments_in_parallel(dtype, c, segment, monkeypatch):
    """Long runs of new tokens are cut into segments that run side by side: with short segments every schedule of the
    other test uses them (sequences of 300, 129 and 3 tokens in one step: eighteen, eight and one segment; pieces that end
    inside a segment; a state that the prompt before left), and with the real segment length a prompt of 1,000 tokens
    beside one of 513 and one of 512."""
    from toyinfer_b200.kernels import recurrent as KR
    m, w, mcfg = make_ssm(dtype, c)
    if segment is not None:
        monkeypatch.setattr(KR, "SSD_SEGMENT", segment)
        lens = [300, 129, 3]
    else:
        lens = [1000, 513, 512]
    xs = inputs(lens, 56, 31, dtype)
    wants = [plain.mamba2(x.double(), w, mcfg, 1e-5) for x in xs]
    if segment is not None:
        check_all_schedules(m, xs, wants, dtype, scale=3.0)
        return
    for sched in ([[(0, 1000), (1, 513), (2, 512)]], [[(0, 40), (1, 1)], [(0, 960), (1, 512), (2, 512)]]):
        got = feed(m, m.memory_request(), xs, sched, dtype, n_slots=3, pre_use=False)
        if dtype == torch.bfloat16:
            # Rounded inputs under decays near one leave a row now and then a tenth away from the exact result, with or
            # without segments; what segments may change is the order of float32 sums, a rounding step of the output.
            monkeypatch.setattr(KR, "SSD_SEGMENT", 10 ** 9)
            wants = feed(m, m.memory_request(), xs, sched, dtype, n_slots=3, pre_use=False)
            monkeypatch.undo()
        for g, x in zip(got, wants):
            torch.testing.assert_close(g, x, **(tol(dtype, 8.0) if dtype == torch.float32 else dict(rtol=2e-2, atol=0.03)))


@pytest.mark.parametrize("dtype", DT)
def test_mamba2_long_decoding_in_a_used_slot(dtype):
    """Four hundred single-token steps after a short prompt: a state that drifts, or a convolution window that slips by
    one, adds up."""
    c = SSM[0]
    m, w, mcfg = make_ssm(dtype, c, seed=9)
    x = inputs([420], 56, 2, dtype)[0]
    want = plain.mamba2(x.double(), w, mcfg, 1e-5)
    sched = [[(0, 20)]] + [[(0, 1)] for _ in range(400)]
    got = feed(m, m.memory_request(), [x], sched, dtype)[0]
    torch.testing.assert_close(got, want, **tol(dtype, 3.0))


@pytest.mark.parametrize("dtype", DT)
def test_attention_long_decoding_across_pages_and_past_the_window(dtype):
    """Three hundred single-token steps: the window passes over decoded tokens and over three page borders."""
    for make, fn, c in ((make_sigmoid, plain.sigmoid_attention, SIGMOID[0]), (make_diff, plain.diff_attention, DIFF[0])):
        m, w, mcfg = make(dtype, c)
        x = loud_inputs(330, 56, 21, [5, 29, 64, 100, 191, 192, 280], 30.0 if dtype == torch.float32 else 6.0).to(dtype)
        want = fn(x.double(), w, mcfg, 1e-5)
        sched = [[(0, 30)]] + [[(0, 1)] for _ in range(300)]
        got = feed(m, m.memory_request(), [x], sched, dtype)[0]
        torch.testing.assert_close(got, want, **tol(dtype, 30.0))
