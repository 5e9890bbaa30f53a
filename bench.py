"""Benchmark of the engine on one B200: decode tokens per second of a Llama-3.1-8B-shaped model with random bf16
weights at batch 8 and 8,192 tokens of context per request, with the 2,048-token prefill, the decode roofline and
decode at batch 1 and 64 on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C] [--no-points]
    python bench.py --workload 3b-serving   # 64 requests of mixed lengths through Engine.admit/step, Llama-3.2-3B shape
    python bench.py --workload 1b-long      # 4 prompts of 32,768 tokens in 2,048-token portions, then 256 sampled steps
    python bench.py --kernels               # single kernels against the library on the layer's shapes
    python bench.py --attention --head-dim 64 --queries 2048 --keys 32768     # the attention kernels alone
    python bench.py --timeline --batch 8    # when the kernels of one layer of a decode step start and end
    python bench.py --impl reference        # the reference arm (unavailable here: it needs JAX and a TPU)

A "step" is one decode step of the whole batch.  `value` is timed on the device with CUDA events around K calls of the
engine's step function (inputs sent from pinned host memory each step, no read-back); `e2e` is the same through the
public entry point (Engine.admit / Engine.step: host token ids in, sampled token ids read back every step).  A decode
step reads more than 16 GB, far over the 126 MB L2, so no flush is needed between steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

POINT_PAUSE_S = 2.0          # idle time before each of the extra points (decode at batch 1 and 64)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


def baseline_config():
    """Sizes of BASELINE.json's configs[2] (the Llama-3.1-8B shape), as a typed configuration."""
    from mashbox_b200.config.llama import LlamaConfig, RopeScaling
    return LlamaConfig(architecture="LlamaForCausalLM", num_layers=32, hidden=4096, num_heads=32, num_kv_heads=8,
                       head_dim=128, intermediate=14336, vocab=128256, rms_eps=1e-5, rope_theta=500000.0,
                       rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 8192), tie_embeddings=False,
                       attention_bias=False, max_position=131072)


class Clocks:
    """Samples nvidia-smi every 200 ms while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.remove(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def flops_prefill(c, layers, n_tokens):
    H, KV, HD, D, F, V = c.num_heads, c.num_kv_heads, c.head_dim, c.hidden, c.intermediate, c.vocab
    per_layer = 2 * n_tokens * (D * (H + 2 * KV) * HD + H * HD * D + 3 * D * F)
    attn = 4 * (n_tokens * (n_tokens + 1) // 2) * HD * H
    return layers * (per_layer + attn) + 2 * D * V


def bytes_decode(c, layers, batch, kv_len):
    H, KV, HD, D, F, V = c.num_heads, c.num_kv_heads, c.head_dim, c.hidden, c.intermediate, c.vocab
    weights = layers * 2 * (D * (H + 2 * KV) * HD + H * HD * D + 3 * D * F) + 2 * D * V
    cache = layers * batch * kv_len * 2 * KV * HD * 2
    return weights + cache


def run_ours(a):
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource

    torch.cuda.set_device(0)
    dev = "cuda:0"
    c = baseline_config()
    layers = a.layers or c.num_layers
    import dataclasses
    cfg = dataclasses.replace(c, num_layers=layers)
    K, W, ctx = a.steps, a.warmup, a.context
    batches = [a.batch] + ([] if a.no_points else [b for b in (1, 64) if b != a.batch])
    max_b = max(batches)
    per_request = -(-(ctx + 1024) // 64) * 64
    pool_tokens = max_b * per_request + 4096
    shapes = architecture(cfg.architecture).stored_tensors(cfg)
    t0 = time.time()
    eng = Engine.from_config(cfg, RandomSource(shapes, 0, torch.bfloat16, dev), dtype="bfloat16", device=dev,
                             page_size=16, max_tokens=pool_tokens, max_requests=max_b, max_tokens_per_step=2048 + max_b,
                             chunk=2048, max_context=per_request, cuda_graphs=not a.no_graphs,
                             options=json.loads(a.options) if a.options else None)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator().manual_seed(1)
    rand_ids = lambda n: torch.randint(0, cfg.vocab, (n,), generator=gen).tolist()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    clocks = Clocks()
    clocks.start()

    # ---- prefill of 2,048 tokens: one step of one fresh request (its first token is sampled in the same step)
    P = a.prefill_tokens
    pre_ms = []
    for i in range(2 + 3):
        rows = eng.admit([dict(ids=rand_ids(P), max_new=1)])
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        eng.step()
        e1.record()
        torch.cuda.synchronize()
        assert rows[0].finish == "length", rows[0].finish
        if i >= 2:
            pre_ms.append(e0.elapsed_time(e1))
    pre = statistics.median(pre_ms)
    pk = peaks()
    tflops = flops_prefill(cfg, layers, P) / (pre / 1e3) / 1e12
    prefill = {"value": P / (pre / 1e3), "tokens": P, "ms": pre, "frac": tflops / pk["bf16_tflops"],
               "tflops": tflops, "frac_of_sustained": tflops / pk["bf16_tflops_sustained"]}

    # ---- decode
    def decode(batch, with_e2e):
        # requests finish their prompts one after the other and decode while the others still prefill: the prompt is
        # shortened by the mean of that head start, so that the mean context in the timed steps is about `ctx`
        chunks = -(-ctx // 2048)
        plen = ctx - 2 * (K + W) - (batch - 1) * chunks // 2 - 2
        rows = eng.admit([dict(ids=rand_ids(plen), max_new=2 * (K + W) + batch * chunks + 16) for _ in range(batch)])
        while any(r.t_first is None for r in rows):
            eng.step()
        res = {}
        if with_e2e:
            for _ in range(W):
                eng.step()
            torch.cuda.synchronize()
            l0 = ops.COUNTERS["launches"]
            e0, e1 = ev(), ev()
            e0.record()
            t0 = time.perf_counter()
            for _ in range(K):
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            ms = max(e0.elapsed_time(e1), wall * 1e3)
            res["e2e"] = {"value": batch * K / (ms / 1e3), "unit": "tokens/s",
                          "h2d_bytes_per_step": eng.runner.inputs.used * 4, "d2h_bytes_per_step": batch * 4 + 4,
                          "ms_per_step": ms / K}
            res["e2e_launches"] = ops.COUNTERS["launches"] - l0
        # the step function alone: fixed next tokens, no read-back inside the timed region
        runner = eng.runner
        live = [r for r in rows if r.finish is None]
        toks = rand_ids(len(live))
        entries = lambda: [(r.rid, [t], [0]) for r, t in zip(live, toks)]
        for _ in range(W):
            runner.step(entries())
        torch.cuda.synchronize()
        l0 = ops.COUNTERS["launches"]
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(K):
            runner.step(entries())
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        runner.check()
        lens = [runner.cache.get(r.rid).length for r in live]
        res.update(value=len(live) * K / (ms / 1e3), ms_per_step=ms / K, launches=ops.COUNTERS["launches"] - l0,
                   kv_len=sum(lens) / len(lens) - K / 2, batch=len(live))
        eng.cancel(rows)
        return res

    def roof(r):
        gbs = bytes_decode(cfg, layers, r["batch"], r["kv_len"]) / (r["ms_per_step"] / 1e3) / 1e9
        return {"ms_per_step": r["ms_per_step"], "mean_kv_len_timed": round(r["kv_len"], 1), "achieved_gbs": gbs,
                "frac": gbs / pk["hbm_gbs"]}

    main = decode(a.batch, True)
    points, detail = {}, {}
    for b in batches[1:]:
        # a pause, so that the power state the measurement before left (the SM clock stays low for a while after a
        # power-capped run) is not part of this one; the point's own clocks are sampled
        torch.cuda.synchronize()
        time.sleep(POINT_PAUSE_S)
        own = Clocks()
        own.start()
        r = decode(b, False)
        ck = own.stop()
        points[f"decode_b{b}"], detail[f"decode_b{b}"] = r["value"], dict(roof(r), sm_mhz=ck["sm_mhz"])
    points[f"decode_b{a.batch}"], detail[f"decode_b{a.batch}"] = main["value"], roof(main)
    clk = clocks.stop()
    nbytes = bytes_decode(cfg, layers, main["batch"], main["kv_len"])
    achieved = nbytes / (main["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tokens/s, Llama-3.1-8B shape, random bf16 weights", "value": main["value"], "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights made on the GPU, uniform random token ids",
        "config": {"model": "llama-3.1-8b-shape", "layers": layers, "layers_of_config": c.num_layers,
                   "hidden": cfg.hidden, "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate, "vocab": cfg.vocab,
                   "global_batch": main["batch"], "seq_len": ctx, "mean_kv_len_timed": round(main["kv_len"], 1),
                   "page_size": 16,
                   "prefill_tokens": P, "parallelism": "single-gpu", "l2": "inputs larger than L2 (no flush)",
                   "cuda_graphs": bool(eng.runner.use_graphs), "peaks": pk["source"], "load_s": round(load_s, 1),
                   "pause_before_points_s": POINT_PAUSE_S},
        "clocks": clk,
        "e2e": {k: main["e2e"][k] for k in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step")},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "points_roofline": detail,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


WORKLOADS = {
    # BASELINE.json configs[3]: continuous batching of 64 requests, prompts U[128, 4096], outputs U[64, 512], greedy
    "3b-serving": dict(model="llama-3.2-3b-shape", layers=28, hidden=3072, heads=24, kv_heads=8, head_dim=128,
                       intermediate=8192, factor=32.0, requests=64, prompt=(128, 4096), new=(64, 512), temperature=0.0),
    # BASELINE.json configs[4]: 4 prompts of 32,768 tokens in 2,048-token portions, then 256 steps at temperature 1.0
    "1b-long": dict(model="llama-3.2-1b-shape", layers=16, hidden=2048, heads=32, kv_heads=8, head_dim=64,
                    intermediate=8192, factor=32.0, requests=4, prompt=(32768, 32768), new=(256, 256), temperature=1.0),
    # the condition of the reference's published single-user rows: one request, 128 new tokens after a warm request
    # (bf16 here, 4- to 8-bit files there); the last has the shape of Falcon3-1B, which its GGUF calls `llama`
    "1b-single": dict(model="llama-3.2-1b-shape", layers=16, hidden=2048, heads=32, kv_heads=8, head_dim=64,
                      intermediate=8192, factor=32.0, requests=1, prompt=(32, 32), new=(128, 128), temperature=0.0),
    "3b-single": dict(model="llama-3.2-3b-shape", layers=28, hidden=3072, heads=24, kv_heads=8, head_dim=128,
                      intermediate=8192, factor=32.0, requests=1, prompt=(32, 32), new=(128, 128), temperature=0.0),
    "8b-single": dict(model="llama-3.1-8b-shape", layers=32, hidden=4096, heads=32, kv_heads=8, head_dim=128,
                      intermediate=14336, factor=8.0, requests=1, prompt=(32, 32), new=(128, 128), temperature=0.0,
                      tied=False),
    "falcon3-1b-single": dict(model="falcon3-1b-shape", layers=18, hidden=2048, heads=8, kv_heads=4, head_dim=256,
                              intermediate=8192, factor=32.0, requests=1, prompt=(32, 32), new=(128, 128),
                              temperature=0.0, vocab=131072),
}


def run_workload(a):
    """A whole workload through the public entry point (Engine.admit / Engine.step, host token ids in, sampled ids read
    back every step): one JSON line with total, prompt and generated tokens per second, what the scheduler and the
    graph cache did, and how much of the wall time the GPU spent inside steps."""
    import random

    import torch
    from mashbox_b200 import ops
    from mashbox_b200.config.llama import LlamaConfig, RopeScaling
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource

    w = WORKLOADS[a.workload]
    torch.cuda.set_device(0)
    dev = "cuda:0"
    layers = a.layers or w["layers"]
    cfg = LlamaConfig(architecture="LlamaForCausalLM", num_layers=layers, hidden=w["hidden"], num_heads=w["heads"],
                      num_kv_heads=w["kv_heads"], head_dim=w["head_dim"], intermediate=w["intermediate"],
                      vocab=w.get("vocab", 128256),
                      rms_eps=1e-5, rope_theta=500000.0, rope_scaling=RopeScaling("llama3", w["factor"], 1.0, 4.0, 8192),
                      tie_embeddings=w.get("tied", True), attention_bias=False, max_position=131072)
    rng = random.Random(a.seed)
    n_req = a.requests or w["requests"]
    plens = [rng.randint(*w["prompt"]) for _ in range(n_req)]
    news = [rng.randint(*w["new"]) for _ in range(n_req)]
    per_request = max(p + n for p, n in zip(plens, news))
    pool = a.pool_tokens or sum(-(-(p + n) // 64) * 64 for p, n in zip(plens, news)) + 4096
    eng = Engine.from_config(cfg, RandomSource(architecture(cfg.architecture).stored_tensors(cfg), 0, torch.bfloat16, dev),
                             dtype="bfloat16", device=dev, page_size=16, max_tokens=pool, max_requests=n_req,
                             max_tokens_per_step=2048 + n_req, chunk=2048, max_context=-(-per_request // 64) * 64,
                             cuda_graphs=not a.no_graphs, options=json.loads(a.options) if a.options else None)
    gen = torch.Generator().manual_seed(a.seed)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=gen).tolist() for n in plens]
    samp = None if w["temperature"] == 0 else dict(temperature=w["temperature"], seed=a.seed)

    # GPU time inside steps: an event before a step's first launch and one after its sampling kernels
    spans = []
    inner = eng._launch

    def timed_launch(prep, before=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st = eng.runner.stats
        was = (st["graph_captures"], st["graph_replays"])
        e0.record()
        f = inner(prep, before)
        e1.record()
        kind = "captured" if st["graph_captures"] > was[0] else "replayed" if st["graph_replays"] > was[1] else "launched"
        spans.append((e0, e1, sum(p.count for p in prep[0]), kind))
        return f

    def once(timed):
        spans.clear()
        rows = eng.admit([dict(ids=p, max_new=n, samp=samp) for p, n in zip(prompts, news)])
        l0 = ops.COUNTERS["launches"]
        before = dict(eng.runner.stats), dict(eng.scheduler.stats)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps, t_first, new_at_first = 0, None, 0
        while eng.busy():
            eng.step()
            steps += 1
            if t_first is None and all(r.t_first is not None or r.finish is not None for r in rows):
                t_first = time.perf_counter()
                new_at_first = sum(len(r.generated) for r in rows)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        gpu_ms = sum(e0.elapsed_time(e1) for e0, e1, _, _ in spans)
        kinds = {}
        for e0, e1, _, kind in spans:
            k = kinds.setdefault(kind, [0, 0.0])
            k[0] += 1
            k[1] = round(k[1] + e0.elapsed_time(e1), 1)
        new = sum(len(r.generated) for r in rows)
        assert all(r.finish == "length" for r in rows), [r.finish for r in rows]
        rs, ss = eng.runner.stats, eng.scheduler.stats
        return dict(wall_s=wall, steps=steps, new_tokens=new, prompt_tokens=sum(plens), gpu_ms_in_steps=gpu_ms,
                    until_all_first_tokens_s=(t_first or t0 + wall) - t0, new_at_first=new_at_first,
                    preemptions=ss["preemptions"] - before[1]["preemptions"],
                    graph_captures=rs["graph_captures"] - before[0]["graph_captures"],
                    graph_replays=rs["graph_replays"] - before[0]["graph_replays"],
                    capture_s=rs["capture_s"] - before[0]["capture_s"], kinds=kinds,
                    launches=ops.COUNTERS["launches"] - l0, deferred=eng.stats["deferred"])

    eng._launch = timed_launch
    clocks = Clocks()
    if a.workload_warm:
        once(False)                      # a first pass loads every kernel and captures the graphs of recurring shapes
    clocks.start()
    r = once(True)
    clk = clocks.stop()
    wall = r["wall_s"]
    decode_s = wall - r["until_all_first_tokens_s"]
    line = {
        "metric": f"generated tokens/s, {a.workload} workload, {w['model']}, random bf16 weights",
        "value": r["new_tokens"] / wall, "unit": "tokens/s", "n_gpus": 1, "steps": r["steps"], "warmup": int(a.workload_warm),
        "ms_per_step": wall * 1e3 / r["steps"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights made on the GPU, seeded uniform random token ids and lengths",
        "config": {"model": w["model"], "layers": layers, "layers_of_config": w["layers"], "hidden": cfg.hidden,
                   "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate, "vocab": cfg.vocab, "requests": n_req,
                   "prompt_tokens": r["prompt_tokens"], "new_tokens": r["new_tokens"], "temperature": w["temperature"],
                   "pool_tokens": pool, "page_size": 16, "chunk": 2048, "seed": a.seed,
                   "cuda_graphs": bool(eng.runner.use_graphs), "parallelism": "single-gpu"},
        "clocks": clk,
        "workload": {"wall_s": wall, "total_tokens_per_s": (r["prompt_tokens"] + r["new_tokens"]) / wall,
                     "prompt_tokens_per_s_until_all_first_tokens": r["prompt_tokens"] / r["until_all_first_tokens_s"],
                     "generated_tokens_per_s_after_that": (None if decode_s <= 0 else
                                                           (r["new_tokens"] - r["new_at_first"]) / decode_s),
                     "until_all_first_tokens_s": r["until_all_first_tokens_s"],
                     "preemptions": r["preemptions"], "graph_captures": r["graph_captures"],
                     "graph_replays": r["graph_replays"], "graph_capture_s": round(r["capture_s"], 3), "steps_and_gpu_ms_by_kind": r["kinds"], "steps_deferred": r["deferred"],
                     "gpu_s_inside_steps": r["gpu_ms_in_steps"] / 1e3,
                     "share_of_wall_outside_steps": 1.0 - r["gpu_ms_in_steps"] / 1e3 / wall},
        "gpu_launches": r["launches"], "impl": "ours",
    }
    print(json.dumps(line))
    return 0


def run_timeline(a):
    """Start and end of every kernel of one decode step inside its captured graph (CUPTI through torch.profiler; no
    ncu): with programmatic dependent launch the kernels of a step overlap, so their durations alone say little; the
    line gives, for one layer in the middle of the model, when each kernel started, when it ended and how long after
    the END of the kernel before it that was.  One JSON line."""
    import dataclasses

    import torch
    from torch.profiler import ProfilerActivity, profile
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource
    dev = "cuda:0"
    c = baseline_config()
    cfg = dataclasses.replace(c, num_layers=a.layers or c.num_layers)
    B, ctx = a.batch, a.context
    per_request = -(-(ctx + 1024) // 64) * 64
    eng = Engine.from_config(cfg, RandomSource(architecture(cfg.architecture).stored_tensors(cfg), 0, torch.bfloat16, dev),
                             dtype="bfloat16", device=dev, page_size=16, max_tokens=B * per_request + 4096, max_requests=B,
                             max_tokens_per_step=2048 + B, chunk=2048, max_context=per_request,
                             options=json.loads(a.options) if a.options else None)
    gen = torch.Generator().manual_seed(1)
    rows = eng.admit([dict(ids=torch.randint(0, cfg.vocab, (ctx - 64,), generator=gen).tolist(), max_new=256) for _ in range(B)])
    while any(r.t_first is None for r in rows):
        eng.step()
    runner = eng.runner
    entries = lambda: [(r.rid, [5], [0]) for r in rows]
    for _ in range(5):
        runner.step(entries())
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            runner.step(entries())
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type.name == "CUDA" and "emcpy" not in e.name and "emset" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    first = max(i for i, e in enumerate(ev) if "embed" in e.name)
    step = ev[first:]
    t0 = step[0].time_range.start
    att = [i for i, e in enumerate(step) if "attn" in e.name]
    lo, hi = att[len(att) // 2], att[len(att) // 2 + 1]
    layer, prev_end = [], step[lo - 1].time_range.end
    for e in step[lo:hi]:
        layer.append({"kernel": e.name.split("(")[0][:60], "start_us": round(e.time_range.start - t0, 1),
                      "end_us": round(e.time_range.end - t0, 1), "after_end_of_previous_us": round(e.time_range.end - prev_end, 1)})
        prev_end = max(prev_end, e.time_range.end)
    tail = [{"kernel": e.name.split("(")[0][:60], "start_us": round(e.time_range.start - t0, 1),
             "end_us": round(e.time_range.end - t0, 1)} for e in step[att[-1] + 1:]]
    print(json.dumps({"impl": "ours", "timeline": {"batch": B, "context": ctx, "layers": cfg.num_layers, "kernels_in_step": len(step),
                                                   "step_us": round(step[-1].time_range.end - t0, 1),
                                                   "layer_us": round(step[hi].time_range.start - step[lo].time_range.start, 1),
                                                   "one_layer": layer, "after_the_last_attention": tail}}))
    return 0


def run_attention(a):
    """Times the attention kernels alone on one layer's cache (one JSON line; also the workload of their ncu captures):
    the prompt form -- a portion of `--queries` tokens at the end of `--keys` tokens of context, tcgen05 kernel against
    the mma.sync kernel -- and the decode form, `--batch` one-token sequences of `--keys` tokens each."""
    import numpy as np
    import torch
    from mashbox_b200 import ops
    dev = "cuda:0"
    H, KV, HD, page = a.heads, a.kv_heads, a.head_dim, 16
    Q, ctx, B = a.queries, a.keys, a.batch
    G = H // KV
    gen = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = ops.new_error_word(dev)

    def timed(f, n):
        for _ in range(3):
            f()
        ts = []
        for _ in range(n):
            flush.zero_()
            e0, e1 = ev(), ev()
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    out = {"config": dict(heads=H, kv_heads=KV, head_dim=HD, page_size=page)}
    # ---- prompt form: one sequence, its last Q tokens are the step's
    pages = -(-ctx // page)
    pool = (torch.randn(2, pages, KV, page, HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    table = torch.randperm(pages, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(dev).reshape(1, pages)
    q = (torch.randn(Q, H * HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    o = torch.empty(Q, H * HD, device=dev, dtype=torch.bfloat16)
    args = (i32([0]), i32([Q]), i32([ctx - Q]))
    zero, none = i32([0]), i32([-1])
    flops = 4.0 * HD * H * sum(min(ctx, ctx - Q + t + 1) for t in range(Q))
    res = {"queries": Q, "keys": ctx}
    if ops.attention_tc5_supports(HD, page):
        rows = ops.attention_tc5_rows()
        items = i32([v for m in range(-(-Q * G // rows) - 1, -1, -1) for v in (0, m, 0, 1)])
        n = items.numel() // 4
        us = timed(lambda: ops.attention_tc5(q, H * HD, o, pool[0], pool[1], items, n, *args, zero, table, H, KV, HD, page,
                                             pages, None, HD ** -0.5, err), a.steps)
        res["tcgen05_us"], res["tcgen05_tflops"] = us, flops / us / 1e6
    items = i32([v for m in range(-(-Q * G // 64) - 1, -1, -1) for v in (0, m, 0, 1)])
    n = items.numel() // 4
    us = timed(lambda: ops.attention_tma(q, H * HD, o, pool[0], pool[1], items, n, False, *args, none, zero, table,
                                         None, None, 1, H, KV, HD, page, pages, None, HD ** -0.5, err), a.steps)
    res["mma_sync_us"], res["mma_sync_tflops"] = us, flops / us / 1e6
    out["prompt_form"] = res
    del pool
    # ---- decode form: B sequences of ctx tokens, one token each, the keys cut into the splits the mixer would choose
    pages = B * -(-ctx // page)
    pool = (torch.randn(2, pages, KV, page, HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(B, -1)
    q = (torch.randn(B, H * HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    o = torch.empty(B, H * HD, device=dev, dtype=torch.bfloat16)
    ns = max(1, min(32, -(-296 // (B * KV)), ctx // 128))
    ns = 1 << (ns.bit_length() - 1)
    items = i32([v for s in range(B) for sp in range(ns) for v in (s, 0, sp, ns)])
    part_o, part_ml = torch.empty(B * H * ns, HD, device=dev), torch.empty(B * H * ns, 2, device=dev)
    rows, ones, last = i32(list(range(B))), i32([1] * B), i32([ctx - 1] * B)
    us = timed(lambda: ops.attention_tma(q, H * HD, o, pool[0], pool[1], items, B * ns, True, rows, ones, last, rows, rows,
                                         table, part_o, part_ml, ns, H, KV, HD, page, pages, None, HD ** -0.5, err,
                                         merge=ns > 1), a.steps)
    nbytes = B * ctx * KV * HD * 2 * 2
    out["decode_form"] = {"batch": B, "keys": ctx, "splits": ns, "us": us, "gbs": nbytes / us / 1e3,
                          "frac_of_hbm_peak": nbytes / us / 1e3 / peaks()["hbm_gbs"]}
    ops.check_error_word(err)
    print(json.dumps({"impl": "ours", "attention": out, "note": "CUDA-event time of single launches after an L2 flush"}))
    return 0


def run_kernels(a):
    """Times this repo's matrix-product and attention kernels next to the library's on the layer shapes of the
    configuration (2,048 tokens and a decode batch), one JSON line; also the workload of the ncu captures of single
    kernels (few launches, under 2 GB on the device)."""
    import torch
    from mashbox_b200 import ops
    dev = "cuda:0"
    c = baseline_config()
    D, F, QKV, V = c.hidden, c.intermediate, (c.num_heads + 2 * c.num_kv_heads) * c.head_dim, c.vocab
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(f, n=a.steps):
        for _ in range(max(3, a.warmup)):
            f()
        ts = []
        for _ in range(n):
            flush.zero_()                                   # L2 is flushed between timed launches
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    out = {}
    T = a.prefill_tokens
    for name, M, K in (("qkv", QKV, D), ("o", D, D), ("gate_up", 2 * F, D), ("down", D, F)):
        x, w = rnd(T, K), rnd(M, K)
        y = torch.empty(T, M, device=dev, dtype=torch.bfloat16)
        own = timed(lambda: ops.linear_tc5(x, w, y, "plain"))
        lib = timed(lambda: torch.mm(x, w.t(), out=y))
        fl = 2 * T * M * K
        out[f"prefill_{name}"] = {"own_us": own, "library_us": lib, "own_tflops": fl / own / 1e6, "library_tflops": fl / lib / 1e6}
    x, w = rnd(T, D), rnd(2 * F, D)
    y = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    out["prefill_gate_up_swiglu_fused"] = {"own_us": timed(lambda: ops.linear_tc5(x, w, y, "swiglu"))}
    # decode batch: every product as a captured graph of launches over different weights (more than the L2 holds), so the
    # figure is the time from launch to launch inside a step; library product against the matrix-vector kernel (at most
    # 4 tokens) and the weight-streaming kernel with its folded forms
    def chained(f, n_w):
        for i in range(n_w):
            f(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n_w):
                f(i)
        g.replay()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / n_w)
        return statistics.median(ts)

    B = a.batch
    for name, M, K in (("o", D, D), ("qkv", QKV, D), ("down", D, F), ("gate_up", 2 * F, D)):
        n_w = max(8, int(600e6 // (M * K * 2)))
        ws = [rnd(M, K) for _ in range(n_w)]
        x, y = rnd(B, K), torch.empty(B, M, device=dev, dtype=torch.bfloat16)
        h = torch.randn(B, K, device=dev, generator=gen)
        hs = torch.randn(B, M, device=dev, generator=gen)
        nw, nw_out = torch.ones(K, device=dev), torch.ones(M, device=dev)
        sums_in = torch.full(((K + 31) // 32, 16), 32.0, device=dev)
        sums_out, scaled_out = torch.empty((M + 31) // 32, 16, device=dev), torch.empty(B, M, device=dev, dtype=torch.bfloat16)
        ops.set_pdl(False)
        r = {"library_us": chained(lambda i: torch.mm(x, ws[i].t(), out=y), n_w),
             "stream_plain_launch_us": chained(lambda i: ops.linear_stream(x, ws[i], y, "plain"), n_w)}
        ops.set_pdl(True)           # from here on as the engine launches them: programmatic dependent launch
        r.update({"stream_us": chained(lambda i: ops.linear_stream(x, ws[i], y, "plain"), n_w),
                  "stream_of_normalised_us": chained(lambda i: ops.linear_stream(x, ws[i], y, "plain", sums_in, 1e-5), n_w),
                  "stream_residual_us": chained(lambda i: ops.linear_stream_residual(x, ws[i], hs, None, sums_out, nw_out, scaled_out), n_w)})
        if B <= 4:
            # the matrix-vector kernels in the forms the engine runs at one token: with the residual add; of the
            # normalised stream (the norm inside the kernel), for gate/up with SwiGLU
            r["gemv_us"] = chained(lambda i: ops.linear_gemv(x, ws[i], y, "plain"), n_w)
            r["gemv_residual_us"] = chained(lambda i: ops.linear_gemv_residual(x, ws[i], hs), n_w)
            if K < 8192 and name != "gate_up":
                r["gemv_of_normalised_us"] = chained(lambda i: ops.linear_gemv_normed(h, nw, 1e-5, ws[i], y), n_w)
            if name == "gate_up":
                act1 = torch.empty(B, F, device=dev, dtype=torch.bfloat16)
                r["gemv_of_normalised_swiglu_us"] = chained(lambda i: ops.linear_gemv_normed(h, nw, 1e-5, ws[i], act1, "swiglu"), n_w)
        if name == "gate_up":
            act, hh = torch.empty(B, F, device=dev, dtype=torch.bfloat16), torch.empty(B, K, device=dev, dtype=torch.bfloat16)
            r["stream_of_normalised_swiglu_us"] = chained(lambda i: ops.linear_stream(x, ws[i], act, "swiglu", sums_in, 1e-5), n_w)
            r["norm_library_gate_us"] = chained(lambda i: (ops.add_rmsnorm(h, None, None, nw, 1e-5, hh, None),
                                                           torch.mm(hh, ws[i].t(), out=y), ops.swiglu(y, act)), n_w)
        r["ideal_us_at_peak"] = M * K * 2 / peaks()["hbm_gbs"] / 1e3
        out[f"decode_b{B}_{name}"] = r
        del ws
    ops.check_error_word(ops.error_word(dev))
    print(json.dumps({"impl": "ours", "kernels": out, "note": "prefill: CUDA-event time of single launches after an L2 flush (launch gaps "
                      "of the Python caller are inside); decode: per launch inside a captured graph of launches over different weights"}))
    return 0


def run_reference(a):
    """The reference arm: mashbox's own engine from baseline/_ref.  mashbox 0.1.15 installs there with --no-deps, but
    its model and engine modules import JAX (not in this image, no network) and it runs on TPU chips."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        import mashbox.runtime.engine  # noqa: F401
        import mashbox.gguf.archs.dense  # noqa: F401
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": f"mashbox's engine cannot be imported here: "
                          f"{type(e).__name__}: {e} (it is a JAX/TPU program; JAX is not installed and there is no network)"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "mashbox imports, but its engine targets TPU chips through JAX "
                      "and has no CUDA path for this metric"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all of them)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel directly (for profilers)")
    ap.add_argument("--options", default="", help="JSON of engine options (kernel choices), for experiments")
    ap.add_argument("--kernels", action="store_true", help="time single kernels against the library instead of the model")
    ap.add_argument("--attention", action="store_true", help="time the attention kernels alone (--heads --kv-heads --head-dim "
                    "--queries --keys --batch)")
    ap.add_argument("--timeline", action="store_true", help="start and end of every kernel of one layer of a decode step "
                    "inside its graph (--batch --context --layers)")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--queries", type=int, default=2048)
    ap.add_argument("--keys", type=int, default=8192)
    ap.add_argument("--workload", default="", choices=("",) + tuple(WORKLOADS),
                    help="run one of the other workloads of the baseline through Engine.admit/step instead")
    ap.add_argument("--requests", type=int, default=0, help="workloads: fewer requests than the workload names")
    ap.add_argument("--pool-tokens", type=int, default=0, help="workloads: size of the cache pool (0: every request fits)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--workload-warm", type=int, default=1, help="workloads: run the workload once untimed first")
    a = ap.parse_args()
    if a.impl == "reference":
        return run_reference(a)
    if a.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this engine runs on ONE GPU; --gpus {a.gpus} is not measured")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.workload:
        return run_workload(a)
    if a.attention:
        return run_attention(a)
    if a.timeline:
        return run_timeline(a)
    return run_kernels(a) if a.kernels else run_ours(a)


if __name__ == "__main__":
    sys.exit(main())
