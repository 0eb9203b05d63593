"""Furitar through the engine against the plain implementation, in float32 and bfloat16: whole
prompts; the last tokens one by one; prompts in portions down to two tokens; batches of unequal
requests against each alone, one batch after another so that slots, pages and state are used
again; decoding far past a ring's length and over many chunk edges; greedy generation through
the generator."""
import pytest
import torch

import plain_furitar as P
from furitar_cases import CASES, make_folder
from helpers import logits_err, random_ids

pytestmark = pytest.mark.gpu

LENGTHS = [37, 5, 131, 64, 1, 65, 11]


@pytest.fixture(scope="module", params=["A", "B", "C", "D"])
def case(request):
    folder = make_folder(request.param)
    cfg, w = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab"], 300 + i) for i, n in enumerate(LENGTHS)]
    plain = [P.forward(cfg, w, ids)[0] for ids in prompts]
    return {"name": request.param, "folder": folder, "cfg": cfg, "w": w, "prompts": prompts,
            "plain": plain}


def _engine(folder, dtype, max_tokens=4096, **kw):
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    return Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=max_tokens, **kw)


def _close(got, want, dtype):
    err, bound = logits_err(got, want, dtype)
    assert err < bound, (err, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(case, dtype):
    eng = _engine(case["folder"], dtype)
    for ids, want in zip(case["prompts"], case["plain"]):
        s = eng.acquire()
        got = eng.step([s], [ids], [list(range(len(ids)))])
        eng.release(s)
        assert got.shape == want.shape
        _close(got, want, dtype)
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(case, dtype):
    eng = _engine(case["folder"], dtype)
    for ids, want in zip(case["prompts"], case["plain"]):
        n = len(ids)
        head = max(1, n - 40)
        s = eng.acquire()
        rows = [eng.step([s], [ids[:head]], [list(range(head))])]
        for t in range(head, n):
            rows.append(eng.step([s], [[ids[t]]], [[0]]))
        eng.release(s)
        _close(torch.cat(rows), want, dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("portion", [2, 3, 7, 63, 64, 65])
def test_prompts_in_portions(case, dtype, portion):
    eng = _engine(case["folder"], dtype)
    for ids, want in zip(case["prompts"][:4], case["plain"][:4]):
        s = eng.acquire()
        rows = []
        for lo in range(0, len(ids), portion):
            part = ids[lo:lo + portion]
            rows.append(eng.step([s], [part], [list(range(len(part)))]))
        eng.release(s)
        _close(torch.cat(rows), want, dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_slots_reused(case, dtype):
    """The prompts' first parts in one step, then one token each; a request that runs out of
    tokens leaves the batch; the next batch starts in the slots, pages and state the first one
    gave back.  Every request's logits equal those it has alone."""
    eng = _engine(case["folder"], dtype, max_tokens=1024, max_seqs=4)
    prompts, plain = case["prompts"], case["plain"]
    for batch in ([0, 1, 2], [3, 4, 5, 6], [2, 0], [6, 2, 4]):
        slots = {r: eng.acquire() for r in batch}
        heads = {r: max(1, len(prompts[r]) - 9) for r in batch}
        got = {r: [] for r in batch}
        out = eng.step([slots[r] for r in batch], [prompts[r][:heads[r]] for r in batch],
                       [list(range(heads[r])) for r in batch])
        at = 0
        for r in batch:
            got[r].append(out[at:at + heads[r]])
            at += heads[r]
        pos = dict(heads)
        live = [r for r in batch if pos[r] < len(prompts[r])]
        while live:
            out = eng.step([slots[r] for r in live], [[prompts[r][pos[r]]] for r in live],
                           [[0]] * len(live))
            for i, r in enumerate(live):
                got[r].append(out[i:i + 1])
                pos[r] += 1
            live = [r for r in live if pos[r] < len(prompts[r])]
        for r in batch:
            _close(torch.cat(got[r]), plain[r], dtype)
            eng.release(slots[r])
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_step_a_new_portion_beside_single_tokens(case, dtype):
    """One request goes on by 20 tokens while two others go on by one, in the same step."""
    eng = _engine(case["folder"], dtype)
    prompts, plain = case["prompts"], case["plain"]
    a, b, c = 2, 0, 6
    sa, sb, sc = eng.acquire(), eng.acquire(), eng.acquire()
    eng.step([sa, sb, sc], [prompts[a][:100], prompts[b][:30], prompts[c][:10]], [[], [], []])
    out = eng.step([sb, sa, sc], [[prompts[b][30]], prompts[a][100:120], [prompts[c][10]]],
                   [[0], list(range(20)), [0]])
    _close(out[0:1], plain[b][30:31], dtype)
    _close(out[1:21], plain[a][100:120], dtype)
    _close(out[21:22], plain[c][10:11], dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_rings_and_over_chunk_edges(dtype):
    """Configuration A keeps rings of a few hundred positions: 420 tokens one by one wrap them
    and cross dozens of chunk edges; the same in portions of 50."""
    folder = make_folder("A")
    cfg, w = P.load_folder(folder)
    ids = random_ids(430, cfg["vocab"], 77)
    want = P.forward(cfg, w, ids)[0]
    eng = _engine(folder, dtype, max_tokens=1024)
    assert all(g.ring and g.ring < 430 for g in eng.cache.groups)
    s = eng.acquire()
    rows = [eng.step([s], [ids[:10]], [list(range(10))])]
    for t in range(10, 430):
        rows.append(eng.step([s], [[ids[t]]], [[0]]))
    eng.release(s)
    _close(torch.cat(rows), want, dtype)
    s = eng.acquire()
    rows = [eng.step([s], [ids[lo:lo + 50]], [list(range(len(ids[lo:lo + 50])))])
            for lo in range(0, 430, 50)]
    _close(torch.cat(rows), want, dtype)
    # a whole prompt longer than the rings, then decoding from what it left
    eng.release(s)
    s = eng.acquire()
    rows = [eng.step([s], [ids[:400]], [list(range(400))])]
    for t in range(400, 430):
        rows.append(eng.step([s], [[ids[t]]], [[0]]))
    _close(torch.cat(rows), want, dtype)
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_a_prompt_of_one(case, dtype):
    """Position 0 alone (no row before it for the shift, one key and the sink), then position 1."""
    eng = _engine(case["folder"], dtype)
    ids, want = case["prompts"][0], case["plain"][0]
    s = eng.acquire()
    a = eng.step([s], [[ids[0]]], [[0]])
    b = eng.step([s], [[ids[1]]], [[0]])
    c = eng.step([s], [ids[2:4]], [[0, 1]])
    _close(torch.cat([a, b, c]), want[:4], dtype)
    # a slot used before starts from zero state again
    eng.release(s)
    s2 = eng.acquire()
    assert s2 == s
    again = eng.step([s2], [[ids[0]]], [[0]])
    _close(again, want[:1], dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_generator(case, dtype):
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = case["cfg"], case["w"]
    prompts = [case["prompts"][i][:20] for i in (0, 1, 3)]
    gen = Generator(Model.from_folder(case["folder"], dtype, "cuda:0"), max_tokens=2048, max_batch=2)
    got = gen.generate(prompts, 12, SamplingParams.greedy(), stop_token_ids=[])
    for p, r in zip(prompts, got):
        assert len(r.tokens) == 12
        if dtype == "float32":
            assert r.tokens == P.generate_greedy(cfg, w, p, 12)
            continue
        # bfloat16: each token is, on the prefix the engine itself produced, the plain
        # implementation's choice or one that rounding can tip it to
        ids = list(p)
        for tok in r.tokens:
            logits = P.forward(cfg, w, ids)[0][-1]
            slack = 0.05 * float(logits.abs().max())
            assert float(logits[tok]) >= float(logits.max()) - slack
            ids.append(tok)


def test_command_line_generates(capsys):
    from minfer_b200 import cli
    folder = make_folder("B")
    cfg, w = P.load_folder(folder)
    rc = cli.main([folder, "5,17,3", "--greedy", "--repeat-penalty", "1.0", "-n", "6",
                   "--dtype", "float32", "--stop", "100000"])
    out = capsys.readouterr().out
    assert rc == 0
    want = P.generate_greedy(cfg, w, [5, 17, 3], 6)
    assert " ".join(str(t) for t in want) in out
    assert "Prefill: 3 tokens" in out and "Generated: 6 tokens" in out


def test_sampled_generation_is_reproducible_and_independent_of_the_batch():
    """Temperature sampling through the generator: the same seed gives the same tokens, alone or
    beside other requests (float32: the logits are the same bits in both)."""
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    folder = make_folder("A")
    cfg, _ = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab"], 900 + n) for n in (12, 30, 5)]
    model = Model.from_folder(folder, "float32", "cuda:0")
    sp = SamplingParams(0.8, 20, 0.95, 1.1, 0.0, 0.0, 1234)
    together = Generator(model, max_tokens=2048, max_batch=3).generate(prompts, 10, sp, stop_token_ids=[])
    again = Generator(model, max_tokens=2048, max_batch=3).generate(prompts, 10, sp, stop_token_ids=[])
    assert [r.tokens for r in together] == [r.tokens for r in again]
    assert all(len(r.tokens) == 10 and all(0 <= t < cfg["vocab"] for t in r.tokens) for r in together)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_process(dtype):
    """``bin/trace_run`` on a Furitar folder: whole prompts, then one request's last tokens one by
    one beside another that ends earlier; logits files against the plain implementation."""
    import json
    import os
    import subprocess
    import sys
    import tempfile
    import numpy as np
    folder = make_folder("D")
    cfg, w = P.load_folder(folder)
    a, b = random_ids(70, cfg["vocab"], 1), random_ids(9, cfg["vocab"], 2)
    plain = {"a": P.forward(cfg, w, a)[0], "b": P.forward(cfg, w, b)[0]}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []}]
    expect = {0: [("a", [0, 59]), ("b", [6])]}
    for i in range(10):
        entries = [{"id": "a", "tokens": [a[60 + i]], "want": [0] if i % 2 == 0 else []}]
        rows = [("a", [60 + i])] if i % 2 == 0 else []
        if i < 2:
            entries.append({"id": "b", "tokens": [b[7 + i]], "want": [0]})
            rows.append(("b", [7 + i]))
        end = (["b"] if i == 1 else []) + (["a"] if i == 9 else [])
        steps.append({"step": i + 1, "entries": entries, "end": end})
        expect[i + 1] = rows
    out = tempfile.mkdtemp()
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder,
                           "--dtype", dtype, "--out", out, "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    for step, rows in expect.items():
        path = os.path.join(out, f"{step}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, cfg["vocab"]))
        want = torch.cat([plain[r][places] for r, places in rows])
        _close(got, want, dtype)
