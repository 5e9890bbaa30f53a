"""-m gpu: the engine through its Python entry point -- greedy and sampled generation against the plain implementation,
long decoding, the first tokens of a sequence, preemption when pages run out, cancelling, the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.plain import llama as plain
from tests.plain import sampling as psamp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(tmp, name, mode, **kw):
    from mashbox_b200.engine.engine import Engine
    dtype, opts = H.MODES[mode]
    folder = H.make_folder(tmp, name, H.store_for(dtype))
    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_requests", 4)
    return folder, Engine.from_folder(folder, dtype=dtype, page_size=H.TINY[name][2], options=opts, **kw)


def teacher_forced_ok(folder, prompt, ids, mode, samp=None):
    """every generated token is what the plain implementation picks from the same history (or, where the plain model
    has a near tie or bfloat16 noise reaches the gap, one of the near-best)"""
    cfg, W = H._plain_model(folder)
    lg = plain.forward(cfg, W, prompt + ids[:-1])[len(prompt) - 1:].numpy()
    noise = 1e-4 if mode == "f32" else 0.03 * np.abs(lg).max()
    for i, (t, row) in enumerate(zip(ids, lg)):
        if samp is None:
            assert row.max() - row[t] <= noise, (i, t, int(row.argmax()), float(row.max() - row[t]))
        else:
            want = psamp.sample(row.astype(np.float32), step=i, **samp)
            if t != want:                # allowed only when the two leading noisy scores are closer than the noise
                x = psamp.transform(row.astype(np.float32), samp["temperature"])
                s = np.array([x[v] + psamp.gumbel(psamp.philox_word(samp["seed"], v, i)) for v in (t, want)])
                assert abs(s[0] - s[1]) <= noise / samp["temperature"], (i, t, want, s)
                assert mode != "f32" or abs(s[0] - s[1]) <= 1e-4


@pytest.mark.parametrize("name,mode", [(n, m) for n in ("A", "B") for m in ("f32", "bf16")])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name, mode):
    folder, eng = engine(tmp_path_factory.mktemp("m"), name, mode)
    prompts = H.prompts_for(name, (7, 13), seed=4)
    out = eng.generate(prompts, max_new=16)
    assert out["finish"] == ["length", "length"] and [len(x) for x in out["ids"]] == [16, 16]
    assert out["timing"]["new_tokens"] == 32 and not out["timing"]["sampled"]
    for p, ids in zip(prompts, out["ids"]):
        teacher_forced_ok(folder, p, ids, mode)
    eng.cache.check()
    assert eng.cache.free_pages() == [eng.cache.num_pages]
    # alone and in the batch: the same tokens
    alone = eng.generate([prompts[1]], max_new=16)
    if mode == "f32":
        assert alone["ids"][0] == out["ids"][1]
    # a stop token ends the answer and is not emitted
    stop = out["ids"][0][5]
    cut = eng.generate([prompts[0]], max_new=16, stop_ids=(stop,))
    first = out["ids"][0].index(stop)
    if mode == "f32":
        assert cut["finish"] == ["stop"] and cut["ids"][0] == out["ids"][0][:first]


@pytest.mark.parametrize("mode", ["f32", "bf16"])
def test_sampled_generation_chunked_and_mixed(tmp_path_factory, mode):
    """configuration B's workload: prompts of 5, 40 and 130 tokens, prompt portions of 32 beside decoded tokens,
    24 tokens each at temperature 0.8 with seed 7"""
    folder, eng = engine(tmp_path_factory.mktemp("m"), "B", mode, chunk=32, max_tokens_per_step=40)
    prompts = H.prompts_for("B", (5, 40, 130), seed=5)
    samp = dict(temperature=0.8, seed=7)
    out = eng.generate(prompts, max_new=24, samp=[samp] * 3)
    assert out["timing"]["sampled"] and [len(x) for x in out["ids"]] == [24, 24, 24]
    for p, ids in zip(prompts, out["ids"]):
        teacher_forced_ok(folder, p, ids, mode, samp)
    assert len({tuple(x) for x in out["ids"]}) == 3
    # other settings reach the kernel too: top_k 1 is greedy whatever the temperature
    g = eng.generate(prompts[:1], max_new=8)
    k1 = eng.generate(prompts[:1], max_new=8, samp=[dict(temperature=1.5, top_k=1, seed=3)])
    assert g["ids"] == k1["ids"]
    # a repetition penalty changes a greedy answer that repeats itself
    rep = eng.generate(prompts[:1], max_new=24, samp=[dict(repetition_penalty=1.8, presence_penalty=0.5)])
    plain_rep = eng.generate(prompts[:1], max_new=24)
    assert len(set(rep["ids"][0])) >= len(set(plain_rep["ids"][0]))


@pytest.mark.parametrize("mode", ["f32", "bf16"])
def test_pages_run_out_preemption_keeps_the_answers(tmp_path_factory, mode):
    tmp = tmp_path_factory.mktemp("m")
    prompts = H.prompts_for("A", (20, 24, 17, 30), seed=6)
    samp = [dict(temperature=0.7, seed=11 + i) for i in range(4)]
    samp[1]["repetition_penalty"] = 1.3          # its penalty state is rebuilt after a preemption: that step waits for
    samp[3]["frequency_penalty"] = 0.4           # the ids still in flight instead of being queued ahead
    _, roomy = engine(tmp, "A", mode, max_tokens=1024)
    want = roomy.generate(prompts, max_new=40, samp=samp)
    assert want["preemptions"] == [0, 0, 0, 0]
    _, tight = engine(tmp, "A", mode, max_tokens=160)                 # 4 x 70 tokens do not fit in 160
    got = tight.generate(prompts, max_new=40, samp=samp)
    assert sum(got["preemptions"]) > 0 and got["finish"] == ["length"] * 4
    if mode == "f32":
        assert got["ids"] == want["ids"]
    else:
        same = sum(a == b for x, y in zip(got["ids"], want["ids"]) for a, b in zip(x, y))
        assert same >= 0.8 * 160
    tight.cache.check()
    assert tight.cache.free_pages() == [tight.cache.num_pages]
    # a request that can never fit is refused alone, before anything runs
    with pytest.raises(ValueError, match="over the context"):
        tight.generate([list(range(100))], max_new=100)
    rows = tight.admit([dict(ids=list(range(100)), max_new=100), dict(ids=[1, 2, 3], max_new=2)])
    assert rows[0].finish == "error" and "over the context" in rows[0].error
    while tight.busy():
        tight.step()
    assert rows[1].finish == "length" and len(rows[1].generated) == 2


def test_stop_tokens_while_the_next_step_is_already_queued(tmp_path_factory):
    """Two steps are in flight, so a stop token is seen one step late: the request must still end exactly there, the
    token queued after it must be dropped, a request waiting for its slot must come in, and nothing may leak.  One
    request stops on its first token, one on the token that is also its max_new-th, one in the middle, one never."""
    _, eng = engine(tmp_path_factory.mktemp("m"), "A", "f32", max_requests=2)
    prompts = H.prompts_for("A", (9, 14, 6, 11), seed=12)
    # tokens that differ from step to step make the test sharper than greedy loops: sample with fixed seeds
    samp = [dict(temperature=0.9, seed=40 + i) for i in range(4)]
    free = eng.generate(prompts, max_new=24, samp=samp)
    assert free["finish"] == ["length"] * 4
    stops = [free["ids"][0][7], free["ids"][1][23], None, free["ids"][3][0]]
    reqs = [dict(ids=p, max_new=24, samp=s, stop_ids=() if st is None else (st,)) for p, s, st in zip(prompts, samp, stops)]
    rows = eng.admit(reqs)
    ended, calls = [], 0
    while eng.busy():
        ended += eng.step()
        calls += 1
        assert calls < 400
    assert sorted(id(r) for r in ended) == sorted(id(r) for r in rows)
    for r, ids, st in zip(rows, free["ids"], stops):
        want = ids if st is None else ids[:ids.index(st)]
        assert r.generated == want and r.finish == ("length" if st is None else "stop"), (r.generated, want, r.finish)
        assert -1 not in r.generated
    eng.cache.check()
    assert eng.cache.free_pages() == [eng.cache.num_pages]
    # and again through generate(), with a token every request stops on somewhere or never
    common = free["ids"][2][10]
    cut = eng.generate(prompts, max_new=24, samp=samp, stop_ids=(common,))
    for got, ids, fin in zip(cut["ids"], free["ids"], cut["finish"]):
        want = ids[:ids.index(common)] if common in ids else ids
        assert got == want and fin == ("stop" if common in ids else "length")
    assert eng.cache.free_pages() == [eng.cache.num_pages]


def test_a_step_that_needs_ids_still_in_flight_waits_for_them(tmp_path_factory):
    """A request whose penalty state has to be rebuilt (what a preemption leaves behind) while its newest token is still
    being sampled cannot be queued ahead: the engine books the step in flight first.  The answer does not change."""
    _, eng = engine(tmp_path_factory.mktemp("m"), "A", "f32")
    prompt = H.prompts_for("A", (8,), seed=3)[0]
    samp = dict(temperature=0.8, seed=5, repetition_penalty=1.4, presence_penalty=0.3)
    want = eng.generate([prompt], max_new=20, samp=[samp])["ids"][0]
    assert eng.stats["deferred"] == 0
    rows = eng.admit([dict(ids=prompt, max_new=20, samp=samp)])
    marked = set()
    while eng.busy():
        n = len(rows[0].generated)
        if n in (5, 11) and n not in marked:
            marked.add(n)
            rows[0].needs_penalty_start = True
        eng.step()
    assert rows[0].generated == want and eng.stats["deferred"] == 2
    assert eng.cache.free_pages() == [eng.cache.num_pages]


@pytest.mark.parametrize("seed,slots,pool,budget,count,burst", [(1, 3, 192, 48, 36, 4), (4, 3, 192, 48, 36, 4),
                                                                 (9, 26, 1600, 96, 70, 30)])
def test_random_traffic_equals_each_request_alone(tmp_path_factory, seed, slots, pool, budget, count, burst):
    """36 requests of random lengths, samplers, stop tokens and arrival times through an engine with three slots, 192
    tokens of cache and 48 tokens a step (portions, preemptions, a few cancellations, two steps in flight all along):
    in float32 every answer is the one the request gets alone in a roomy engine, cut at its stop token.  The third case
    has 26 slots and 70 requests arriving in bursts of up to 30: decode batches of more than 16, which are filled up to
    the grid of sizes and replayed from graphs."""
    import random
    rng = random.Random(seed)
    folder, roomy = engine(tmp_path_factory.mktemp("m"), "A", "f32", max_tokens=512, max_requests=2)
    vocab = H.TINY["A"][0].vocab

    def samp():
        if rng.random() < 0.3:
            return None
        d = dict(temperature=rng.choice([0.5, 0.9, 1.3]), seed=rng.randrange(1 << 40))
        if rng.random() < 0.4: d["top_k"] = rng.choice([1, 5, 40])
        if rng.random() < 0.4: d["top_p"] = rng.choice([0.3, 0.8, 0.95])
        if rng.random() < 0.2: d["min_p"] = 0.05
        if rng.random() < 0.3: d["repetition_penalty"] = 1.2
        if rng.random() < 0.2: d["frequency_penalty"] = 0.3
        return d

    reqs = [dict(ids=[rng.randrange(vocab) for _ in range(rng.randint(1, 70))], max_new=rng.randint(1, 36), samp=samp())
            for _ in range(count)]
    alone = [roomy.generate([q["ids"]], max_new=q["max_new"], samp=[q["samp"]])["ids"][0] for q in reqs]
    for q, a in zip(reqs, alone):
        if rng.random() < 0.35 and a:
            q["stop_ids"] = (a[rng.randrange(len(a))],)
    want = [a[:a.index(q["stop_ids"][0])] if q.get("stop_ids") else a for q, a in zip(reqs, alone)]
    from mashbox_b200.engine.engine import Engine
    tight = Engine.from_folder(folder, dtype="float32", page_size=H.TINY["A"][2], max_tokens=pool, max_requests=slots,
                               max_tokens_per_step=budget, chunk=32)
    seen_batches = []
    inner_prepare = tight.runner.prepare

    def watching_prepare(entries, *a, **k):
        ctx = inner_prepare(entries, *a, **k)
        seen_batches.append((len(entries), ctx.S))
        return ctx
    tight.runner.prepare = watching_prepare
    rows, pending, cancelled, steps = {}, list(range(len(reqs))), set(), 0
    while pending or tight.busy():
        if pending and (rng.random() < 0.3 or not tight.busy()):
            n = rng.randint(1, burst)
            take, pending = pending[:n], pending[n:]
            for i, r in zip(take, tight.admit([reqs[i] for i in take])):
                rows[i] = r
        if rng.random() < 0.03:
            live = [i for i, r in rows.items() if r.finish is None and i not in cancelled]
            if live:
                i = live[rng.randrange(len(live))]
                cancelled.add(i)
                tight.cancel([rows[i]])
        tight.step()
        steps += 1
        assert steps < 20000
    for i, r in rows.items():
        assert -1 not in r.generated
        if r.finish == "cancel":
            assert r.generated == want[i][:len(r.generated)]
        else:
            assert r.generated == want[i], (i, r.finish, reqs[i].get("samp"), reqs[i].get("stop_ids"), r.preemptions)
            assert r.finish == ("stop" if reqs[i].get("stop_ids") else "length")
    tight.cache.check()
    assert tight.cache.free_pages() == [tight.cache.num_pages]
    if slots > 16:
        assert any(real > 16 and filled > real for real, filled in seen_batches), "no decode batch was filled up"
        assert tight.runner.stats["graph_replays"] > 0


def test_cancel_through_on_step(tmp_path_factory):
    _, eng = engine(tmp_path_factory.mktemp("m"), "A", "f32")
    prompts = H.prompts_for("A", (9, 9), seed=7)
    out = eng.generate(prompts, max_new=30, on_step=lambda ids, fin: [0] if len(ids[0]) >= 4 and fin[0] is None else [])
    assert out["finish"] == ["cancel", "length"] and 4 <= len(out["ids"][0]) < 30 and len(out["ids"][1]) == 30
    assert eng.cache.free_pages() == [eng.cache.num_pages]


@pytest.mark.parametrize("name,mode", [("A", "f32"), ("B", "f32"), ("B", "bf16-plain"), ("A", "bf16")])
def test_long_decoding_and_first_tokens(tmp_path_factory, name, mode):
    """a short prompt, then 330 tokens one by one (many pages, a second request decoding beside it part of the time);
    and sequences of one, two and three tokens"""
    from mashbox_b200.engine.replay import make_runner, run_step
    tmp = tmp_path_factory.mktemp("m")
    dtype, opts = H.MODES[mode]
    folder = H.make_folder(tmp, name, H.store_for(dtype))
    runner = make_runner(folder, dtype, 448, page_size=H.TINY[name][2], options=opts)
    long, side = H.prompts_for(name, (335, 90), seed=8)
    got, got_side = [], []
    for i in range(len(long)):
        entries = [dict(id="long", tokens=long[:5] if i == 4 else [long[i]], want=[4] if i == 4 else [0])] if i >= 4 else []
        if 100 <= i < 100 + len(side):
            entries.append(dict(id="side", tokens=[side[i - 100]], want=[0]))
        if not entries:
            continue
        r = run_step(runner, dict(step=i, entries=entries, end=["side"] if i == 100 + len(side) - 1 else [])).numpy()
        got.append(r[0])
        if len(entries) == 2:
            got_side.append(r[1])
    H.check(np.stack(got), folder, long, mode, "long decoding", slice(4, None))
    H.check(np.stack(got_side), folder, side, mode, "decoding beside it")
    run_step(runner, dict(step=0, entries=[], end=["long"]))
    for n in (1, 2, 3):
        p = H.prompts_for(name, (n,), seed=20 + n)[0]
        r = run_step(runner, dict(step=0, entries=[dict(id="s", tokens=p, want=list(range(n)))], end=["s"])).numpy()
        H.check(r, folder, p, mode, f"a sequence of {n}")
    runner.cache.check()


def test_command_line(tmp_path):
    folder = H.make_folder(tmp_path, "A", "float32")
    cmd = [sys.executable, "-m", "mashbox_b200", "run", folder, "--prompt-ids", "5,17,3,200", "--max-tokens", "6",
           "--dtype", "float32", "--ctx", "256"]
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(x) for x in r.stdout.strip().split(",")]
    cfg, W = plain.read_model(folder)
    assert ids == plain.greedy(cfg, W, [5, 17, 3, 200], 6)
    events = [json.loads(l) for l in r.stderr.splitlines() if l.startswith("{")]
    assert [e["event"] for e in events if e["event"] in ("loaded", "warm", "done")] == ["loaded", "warm", "done"]
    assert events[-1]["new_tokens"] == 6 and "lh" not in events[-1]
    # --no-warm answers at once; --trace adds the logit hashes; --cache-dir says where the compiled kernels go
    cache = tmp_path / "kernels"
    t = subprocess.run(cmd + ["--no-warm", "--trace", "--cache-dir", str(cache)], capture_output=True, text=True, env=env,
                       timeout=900)
    assert t.returncode == 0, t.stderr[-2000:]
    assert t.stdout == r.stdout
    events = [json.loads(l) for l in t.stderr.splitlines() if l.startswith("{")]
    assert "warm" not in [e["event"] for e in events] and len(events[-1]["lh"]) == 6
    assert any(f.endswith(".so") for f in os.listdir(cache))
    s = subprocess.run(cmd[:-4] + ["--temperature", "0.8", "--seed", "7", "--top-k", "50", "--dtype", "float32", "--ctx", "256"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert s.returncode == 0 and len(s.stdout.strip().split(",")) == 6
    bad = subprocess.run(cmd[:5] + ["--prompt-ids", "5,999"], capture_output=True, text=True, env=env, timeout=600)
    assert bad.returncode == 2 and "token ids must be 0..255" in bad.stderr


def test_command_line_with_a_tokenizer(tmp_path):
    """--prompt TEXT: tokenizer.json of the folder turns text into ids and ids back into text"""
    import shutil
    from tokenizers import Tokenizer, models, pre_tokenizers
    folder = H.make_folder(tmp_path, "A", "float32")
    words = {f"w{i}": i for i in range(256)}
    tok = Tokenizer(models.WordLevel(vocab=words, unk_token="w0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(folder, "tokenizer.json"))
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "mashbox_b200", "run", folder, "--prompt", "w5 w17 w3 w200", "--max-tokens", "5",
           "--dtype", "float32"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, W = plain.read_model(folder)
    want = plain.greedy(cfg, W, [5, 17, 3, 200], 5)
    assert r.stdout.split() == [f"w{t}" for t in want]
    os.remove(os.path.join(folder, "tokenizer.json"))
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 2 and "tokenizer.json" in r.stderr


@pytest.mark.parametrize("where", ["launch", "wait", "prepare"])
def test_a_step_that_fails_on_the_host_ends_every_live_request_and_leaves_the_engine_usable(tmp_path_factory, where,
                                                                                             monkeypatch):
    """The failure is made on the host (a patched method raises on its n-th call); nothing on the GPU faults.  Three
    requests are live and a step is in flight when it happens.  Every live request ends "error" with the reason,
    no request keeps a placeholder among its ids, the step in flight is forgotten, every page, row and state slot is
    back, and the next generate() gives the answers of an engine that never failed
    (the reference drops its live rows after a failed device call, src/mashbox/runtime/engine.py:752-762)."""
    from mashbox_b200.engine.runner import ModelRunner
    from mashbox_b200.sampling.sampler import Sampler
    folder, eng = engine(tmp_path_factory.mktemp("m"), "A", "f32", chunk=16, max_tokens_per_step=24)
    prompts = H.prompts_for("A", (30, 9, 21), seed=9)
    want = eng.generate(prompts, max_new=3 if where != "wait" else 12)
    target = {"launch": (ModelRunner, "launch"), "wait": (Sampler, "wait"), "prepare": (ModelRunner, "prepare")}[where]
    original = getattr(*target)
    calls = {"n": 0}

    def failing(self, *a, **kw):
        calls["n"] += 1
        if calls["n"] == 5:
            raise RuntimeError("injected on the host")
        return original(self, *a, **kw)

    monkeypatch.setattr(target[0], target[1], failing)
    rows = eng.admit([dict(ids=p, max_new=3 if i == 1 and where != "wait" else 12) for i, p in enumerate(prompts)])
    with pytest.raises(RuntimeError, match="injected on the host"):
        while eng.busy():
            eng.step()
    monkeypatch.setattr(target[0], target[1], original)
    assert calls["n"] == 5
    assert not eng.busy() and eng._flight is None
    assert all(r.finish in ("error", "length") for r in rows) and sum(r.finish == "error" for r in rows) >= 2
    for r in rows:
        assert eng.PLACEHOLDER not in r.generated
        if r.finish == "error":
            assert "injected on the host" in r.error
        else:
            assert len(r.generated) == r.max_new
    eng.cache.check()
    assert eng.cache.free_pages() == [eng.cache.num_pages] and eng.cache.rows.n_free == eng.cache.max_requests
    assert not eng.scheduler.running and not eng.scheduler.waiting
    again = eng.generate(prompts, max_new=3 if where != "wait" else 12)
    assert again["ids"] == want["ids"] and again["finish"] == want["finish"]


def test_traced_generation_gives_the_same_hashes_alone_and_batched(tmp_path_factory):
    """trace=True: generate() returns per generated token the hash of its logits and the top-2 gap.  On the 32-bit path
    a request's hashes are the same alone, in a batch of four with prompt portions beside decoded tokens, and after a
    preemption: the logits are bit-identical, not merely close."""
    from mashbox_b200.engine.engine import Engine
    tmp = tmp_path_factory.mktemp("m")
    folder = H.make_folder(tmp, "B", "float32")
    prompts = H.prompts_for("B", (5, 40, 130, 61), seed=12)
    make = lambda tokens, **kw: Engine.from_folder(folder, dtype="float32", page_size=8, max_tokens=tokens, max_requests=4,
                                                   chunk=32, max_tokens_per_step=40, trace=True, **kw)
    eng = make(1024)
    batched = eng.generate(prompts, max_new=20)
    assert [len(x) for x in batched["lh"]] == [20] * 4
    assert all(isinstance(h, int) and 0 <= h < 1 << 32 and g >= 0.0 for row in batched["lh"] for h, g in row)
    for i, p in enumerate(prompts):
        alone = eng.generate([p], max_new=20)
        assert alone["ids"][0] == batched["ids"][i]
        assert alone["lh"][0] == batched["lh"][i], f"request {i}: logits differ in some bit between alone and batched"
    tight = make(264)                                                  # 4 requests of up to 150 tokens do not fit
    squeezed = tight.generate(prompts, max_new=20)
    assert sum(squeezed["preemptions"]) > 0
    assert squeezed["lh"] == batched["lh"] and squeezed["ids"] == batched["ids"]
    # without tracing the result has no "lh" key
    folder2, plain_eng = engine(tmp, "A", "f32")
    assert "lh" not in plain_eng.generate(H.prompts_for("A", (7,)), max_new=2)


@pytest.mark.parametrize("name,mode", [("B", "f32"), ("D", "bf16"), ("A", "f32")])
def test_decode_batches_filled_up_to_a_grid_share_graphs_and_change_nothing(tmp_path, name, mode):
    """Decode batches of 17 to 20 sequences run as batches of 20 (the rest are one-token sequences on the cache's spare
    page, whose results are dropped): one captured graph serves all four sizes, the logits of the real sequences are
    the same bits as without the filling (float32; bfloat16: the same tokens' logits within the test's bars, since a
    library product of 20 rows need not round as one of 17), and the bookkeeping never sees the spare page."""
    from mashbox_b200.engine.loading import load_model
    from mashbox_b200.config.engine import EngineConfig
    from mashbox_b200.engine.runner import ModelRunner
    dtype, opts = H.MODES[mode]
    folder = H.make_folder(tmp_path, name, H.store_for(dtype))
    page = H.TINY[name][2]
    prompts = H.prompts_for(name, tuple(8 + 2 * i for i in range(20)), seed=9)
    SIZES = (20, 19, 18, 17, 18, 20)

    def run(options):
        cfg = EngineConfig(dtype=dtype, page_size=page, max_tokens=20 * 128, max_requests=24, max_tokens_per_step=1024,
                           chunk=1024, device="cuda:0")
        runner = ModelRunner(load_model(folder, dtype=dtype, device="cuda:0"), cfg, dict(opts, **options))
        for i in range(20):
            runner.cache.admit(i)
        runner.step([(i, p[:-6], []) for i, p in enumerate(prompts)])
        fed = [len(p) - 6 for p in prompts]
        got = []
        for live in SIZES:                                             # each size of the grid cell, two of them twice
            lg = runner.step([(i, [prompts[i][fed[i]]], [0]) for i in range(live)])
            assert lg.shape[0] == live
            for i in range(live):
                fed[i] += 1
            got.append((lg.float().cpu().numpy(), list(fed)))
        runner.check()
        for i in range(20):
            runner.cache.release(i)
        runner.cache.check()
        assert all(f == runner.cache.num_pages for f in runner.cache.free_pages())
        return got, runner.stats

    filled, st = run({})
    exact, st0 = run({"fill_decode_batches": False})
    # sizes 20, 19, 18, 17, 18, 20: filled, all six steps have one shape (the first sizes the buffers, the second is the
    # first of its shape with those buffers, the third is captured, three replays); unfilled, only 18 comes twice
    # after the first step and nothing is replayed
    assert (st["graph_captures"], st["graph_replays"]) == (1, 3), st
    assert (st0["graph_captures"], st0["graph_replays"]) == (1, 0), st0
    for (a, fed), (b, _), live in zip(filled, exact, SIZES):
        if mode == "f32":
            assert np.array_equal(a, b)
        for i in (0, live - 1):
            H.check(a[i:i + 1], folder, prompts[i][:fed[i]], mode, f"filled batch of {live}, row {i}", slice(-1, None))


def test_many_step_shapes_graphs_are_replaced_and_everything_finishes(tmp_path):
    """600 requests of random lengths arriving in bursts at an engine with 40 slots: more step shapes than the runner
    keeps graphs for (64), so graphs are captured, replayed and given up all along; every request ends with exactly
    the tokens it asked for, and the cache is whole afterwards."""
    import random
    from mashbox_b200.engine.engine import Engine
    rng = random.Random(3)
    folder = H.make_folder(tmp_path, "C", "bfloat16")
    vocab = H.TINY["C"][0].vocab
    eng = Engine.from_folder(folder, dtype="bfloat16", page_size=H.TINY["C"][2], max_tokens=40 * 320, max_requests=40,
                             max_tokens_per_step=256, chunk=128, max_context=320)
    reqs = [dict(ids=[rng.randrange(vocab) for _ in range(rng.randint(1, 200))], max_new=rng.randint(1, 100),
                 samp=None if rng.random() < 0.5 else dict(temperature=0.8, seed=rng.randrange(1 << 30),
                                                           top_k=rng.choice([0, 20])))
            for _ in range(600)]
    pending, rows, steps = list(range(len(reqs))), {}, 0
    while pending or eng.busy():
        if pending and (rng.random() < 0.25 or not eng.busy()):
            n = rng.randint(1, 25)
            take, pending = pending[:n], pending[n:]
            for i, r in zip(take, eng.admit([reqs[i] for i in take])):
                rows[i] = r
        eng.step()
        steps += 1
        assert steps < 100000
    for i, r in rows.items():
        assert r.finish == "length" and len(r.generated) == reqs[i]["max_new"] and -1 not in r.generated, (i, r.finish)
        assert all(0 <= t < vocab for t in r.generated)
    st = eng.runner.stats
    assert st["graph_captures"] > eng.runner.MAX_GRAPHS and len(eng.runner.graphs) <= eng.runner.MAX_GRAPHS
    assert st["graph_replays"] > 0
    eng.cache.check()
    assert eng.cache.free_pages() == [eng.cache.num_pages]
