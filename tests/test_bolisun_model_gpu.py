"""Whole Bolisun models of several shapes through the engine against the plain implementation: whole prompts,
token-by-token decoding (long enough for states to decay, for windows to pass over decoded tokens and for kept first
positions to be the only old keys left), prompts in pieces down to two tokens and unequal batches under a random schedule
with slots handed back and reused, the sum of the streams after every layer run, greedy generation through the public entry
point, the trace runner and the command line."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from bolisun_cases import CASES, assert_close_logits, prompts, read_folder, write_folder
from conftest import ROOT
from helpers import run_random_schedule
from plain import bolisun_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_folder(name, str(tmp_path_factory.mktemp(f"bolisun_{name}"))) for name in CASES}


_plain = {}


def plain_logits(folder, ids):
    key = (folder, tuple(ids))
    if key not in _plain:
        if folder not in _plain:
            _plain[folder] = read_folder(folder)
        w, cfg = _plain[folder]
        _plain[key] = plain.forward(cfg, w, ids)[0]
    return _plain[key]


def engine(folder, dtype, **kw):
    from toyinfer_b200.engine import Engine
    kw.setdefault("max_tokens", 4096)
    kw.setdefault("max_batch", 8)
    kw.setdefault("max_seq_len", 512)
    return Engine.from_folder(folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompts_of_unequal_lengths_in_one_step(folders, name, dtype):
    eng = engine(folders[name], dtype)
    ids = prompts(name, [1, 2, 65, 140, 7], seed=1)
    slots = [eng.new_sequence() for _ in ids]
    got = eng.step(list(zip(slots, ids)), [list(range(len(x))) for x in ids]).clone()
    if dtype == "float32":
        o = 0
        for x in ids:
            assert_close_logits(got[o:o + len(x)], plain_logits(folders[name], x), dtype, f"{name} prompt of {len(x)}")
            o += len(x)
    else:
        assert_close_logits(got, torch.cat([plain_logits(folders[name], x) for x in ids]), dtype, f"{name} prompts")


@pytest.mark.parametrize("name", list(CASES))
def test_stream_sums_after_every_layer_run(folders, name):
    """The sum of the streams after each scheduled layer (the pending update included), in 32-bit, against the plain
    implementation's: a fault shows in the layer that makes it."""
    from toyinfer_b200.kernels import hyper
    eng = engine(folders[name], "float32")
    ids = prompts(name, [77], seed=9)[0]
    w, cfg = read_folder(folders[name])
    want = plain.forward(cfg, w, ids)[1]
    seen = []
    for blk in eng.model.blocks:
        def wrapped(h, delta, batch, mem, shared, orig=blk.forward, blk=blk):
            h, d = orig(h, delta, batch, mem, shared)
            rows = torch.arange(h.shape[0], dtype=torch.int32, device=h.device)
            seen.append(hyper.hyper_norm(h, d, None, None, 0.0, torch.float32, blk.streams, rows=rows, want_sum=True)[1].cpu())
            return h, d
        blk.forward = wrapped
    s = eng.new_sequence()
    eng.step([(s, ids)])
    assert len(seen) == len(want) == len(cfg["layers"])
    for i, got in enumerate(seen):
        torch.testing.assert_close(got.double(), want[i], rtol=2e-4, atol=2e-4, msg=lambda m: f"{name} layer run {i}: {m}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_prompt_then_token_by_token(folders, name, dtype):
    """Three sequences decode together after prompts of unequal lengths (the longest for 120 steps: every window of these
    models passes over decoded tokens, and a page border is crossed); the shortest ends early; afterwards its slot and
    pages serve a new request as if it were alone."""
    eng = engine(folders[name], dtype)
    ids = prompts(name, [190, 71, 9], seed=2)
    heads = [70, 40, 3]
    want = [plain_logits(folders[name], x) for x in ids]
    slots = [eng.new_sequence() for _ in ids]
    got = eng.step([(s, x[:h]) for s, x, h in zip(slots, ids, heads)], [[h - 1] for h in heads]).clone()
    rows = [[got[i:i + 1]] for i in range(3)]
    fed = list(heads)
    live = [0, 1, 2]
    while live:
        got = eng.step([(slots[i], [ids[i][fed[i]]]) for i in live]).clone()
        for r, i in enumerate(live):
            rows[i].append(got[r:r + 1])
            fed[i] += 1
        for i in list(live):
            if fed[i] == len(ids[i]):
                eng.end_sequence(slots[i])
                live.remove(i)
    for i in range(3):
        assert_close_logits(torch.cat(rows[i]), want[i][heads[i] - 1:], dtype, f"{name} sequence {i} from token {heads[i] - 1}")
    again = prompts(name, [90], seed=3)[0]
    s = eng.new_sequence()
    assert s in slots
    got = eng.step([(s, again)], [list(range(90))])
    assert_close_logits(got, plain_logits(folders[name], again), dtype, f"{name} in a reused slot")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_decoding_from_the_first_token(folders, name, dtype):
    """A sequence fed one token at a time from its very first (the states start at zero, the only key is the token
    itself), without captured graphs and with them."""
    ids = prompts(name, [75], seed=7)[0]
    want = plain_logits(folders[name], ids)
    for graphs in (False, True):
        eng = engine(folders[name], dtype, use_cuda_graph=graphs)
        s = eng.new_sequence()
        rows = [eng.step([(s, [tok])]).clone() for tok in ids]
        assert_close_logits(torch.cat(rows), want, dtype, f"{name} graphs={graphs}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_random_schedule_of_pieces_and_batches(folders, name, dtype):
    eng = engine(folders[name], dtype, n_slots=4)
    ids = prompts(name, [130, 67, 1, 5, 100, 64, 33], seed=4)
    got = run_random_schedule(eng, ids, random.Random(11), max_live=4)
    if dtype == "float32":
        for x, g in zip(ids, got):
            assert_close_logits(g, plain_logits(folders[name], x), dtype, f"{name} request of {len(x)}")
    else:
        assert_close_logits(torch.cat(got), torch.cat([plain_logits(folders[name], x) for x in ids]), dtype, f"{name} requests")
    assert eng.cache.slots.n_free == 4


@pytest.mark.parametrize("name", ["P", "Q"])
def test_pieces_of_two_tokens_and_other_sizes(folders, name):
    """One prompt fed in pieces of 2, 3, 64, 1, 66, ... tokens (an attention window, the kept first positions and a page
    straddle the cuts) gives what the whole prompt gives."""
    eng = engine(folders[name], "float32")
    ids = prompts(name, [200], seed=8)[0]
    want = plain_logits(folders[name], ids)
    s = eng.new_sequence()
    fed, sizes = 0, [2, 3, 64, 1, 66, 2, 2, 5, 100]
    for n in sizes:
        n = min(n, len(ids) - fed)
        if n <= 0:
            break
        got = eng.step([(s, ids[fed:fed + n])], [list(range(n))])
        assert_close_logits(got, want[fed:fed + n], "float32", f"{name} piece at {fed} of {n}")
        fed += n


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_public_entry(folders, name):
    from toyinfer_b200 import LLM, SamplingParams
    llm = LLM(folders[name], dtype="float32", max_seq_len=256, max_batch=4)
    ids = prompts(name, [12, 40, 3], seed=5)
    out = llm.generate(ids, SamplingParams(temperature=0.0), max_new_tokens=24)
    w, cfg = read_folder(folders[name])
    for x, r in zip(ids, out):
        toks = list(r.tokens)
        assert len(toks) == 24
        seq = list(x)
        for t in toks:
            logits = plain.forward(cfg, w, seq)[0][-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3:         # a near tie may fall either way
                assert int(torch.argmax(logits)) == t, (name, len(seq))
            seq.append(t)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_on_a_folder(folders, tmp_path, dtype):
    name = "Q"
    V = CASES[name]["vocab"]
    a, b = prompts(name, [100, 37], seed=6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:90], "want": [0, 89]}, {"id": "b", "tokens": b[:30], "want": [29]}], "end": []}]
    for k in range(10):
        e = [{"id": "a", "tokens": [a[90 + k]], "want": [0]}]
        if k < 7:
            e.append({"id": "b", "tokens": [b[30 + k]], "want": [0] if k % 2 else []})
        steps.append({"step": k + 1, "entries": e, "end": (["b"] if k == 6 else []) + (["a"] if k == 9 else [])})
    out = str(tmp_path)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", dtype, "--out", out,
           "--max-tokens", "256"]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {s['step']}"
    p.stdin.close()
    assert p.wait(timeout=120) == 0
    wa, wb = plain_logits(folders[name], a), plain_logits(folders[name], b)
    read = lambda n: torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
    got, want = [read(0)], [wa[0], wa[89], wb[29]]
    for k in range(10):
        got.append(read(k + 1))
        want += [wa[90 + k]] + ([wb[30 + k]] if (k < 7 and k % 2) else [])
    assert [g.shape[0] for g in got] == [3] + [2 if (k < 7 and k % 2) else 1 for k in range(10)]
    assert_close_logits(torch.cat(got), torch.stack(want), dtype, "all steps")


@pytest.mark.parametrize("name", ["P", "S"])
def test_prompt_shapes_that_come_back_run_from_a_captured_step(folders, name):
    """The same shape of prompt step four times, in other slots each time and with other tokens: from the third time on the
    engine replays a captured graph (states zeroed at hand-out, slots and tokens read on the device, spare rows nobody's),
    and every run gives what the plain implementation gives."""
    eng = engine(folders[name], "float32")
    assert eng.prompt_graph_tokens > 0
    held = []
    for rep in range(4):
        ids = prompts(name, [40, 17], seed=20 + rep)
        slots = [eng.new_sequence() for _ in ids]
        got = eng.step(list(zip(slots, ids))).clone()
        for i, x in enumerate(ids):
            assert_close_logits(got[i:i + 1], plain_logits(folders[name], x)[-1:], "float32", f"{name} run {rep} prompt {i}")
        nxt = [3 + rep, 5]
        got = eng.step([(s, [t]) for s, t in zip(slots, nxt)]).clone()
        for i, x in enumerate(ids):
            assert_close_logits(got[i:i + 1], plain_logits(folders[name], list(x) + [nxt[i]])[-1:], "float32", f"{name} run {rep} next {i}")
        if rep % 2:
            for s in slots:
                eng.end_sequence(s)
        else:
            held.extend(slots)
    assert eng.graph_replays >= 2


def test_command_line_generates_from_a_folder(folders):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "toyinfer"), "--model_dir", folders["R"], "--dtype", "float32", "--max_seq_len", "128",
           "--prompt_ids", "5,6,7;8,9", "--max_new_tokens", "6", "--temperature", "0"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    first = json.loads(r.stdout.strip().splitlines()[0])
    assert first["request"] == 0 and len(first["tokens"]) == 6
    w, cfg = read_folder(folders["R"])
    seq = [5, 6, 7]
    for t in first["tokens"]:
        logits = plain.forward(cfg, w, seq)[0][-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) > 1e-3:
            assert int(torch.argmax(logits)) == t, len(seq)
        seq.append(t)
