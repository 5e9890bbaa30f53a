"""Trace replay: feeds given token ids through the model step by step and writes logits; it samples nothing.

It drives the engine's own model, step function, cache manager and kernels -- the ones generation uses -- and has no
forward pass, cache or loader of its own.  Steps come as JSON lines:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: each request's next tokens and the places among them whose logits are wanted; all entries of a step are one
batch.  `end`: requests finished after the step; their pages are given back.  For a step that wants something the
logits are written to <out>/<step>.f32 as little-endian float32 [wanted, vocab], in the order of the entries and of
`want`; after every step a line `done <step>` is printed and flushed.  With --trace a step that wants something
also writes <out>/<step>.lh.json: per wanted row [hash, gap], the order-independent hash of the row's logits
(sum of bits(lg[v]) * (2 v + 1) mod 2^32) and the gap between its two largest, computed on the device as
mashbox-labs/mashbox traces them (src/mashbox/runtime/engine.py:80-89).
"""
import json
import os
import sys

from ..config.engine import EngineConfig
from .loading import load_model
from .runner import ModelRunner

LIVE_REQUESTS = 8


def make_runner(model_dir, dtype, max_tokens, page_size=16, device="cuda:0", options=None, log=None):
    """max_tokens: the most tokens live requests hold at any time, each request rounded up to a multiple of 64; the
    pool is made for exactly this many, so pages are used again."""
    tokens = -(-int(max_tokens) // 64) * 64
    cfg = EngineConfig(dtype=dtype, page_size=page_size, max_tokens=tokens, max_requests=LIVE_REQUESTS,
                       max_tokens_per_step=max(tokens, 64), chunk=max(tokens, 64), device=device)
    model = load_model(model_dir, dtype=dtype, device=device, log=log)
    return ModelRunner(model, cfg, options)


def run_step(runner, step, out_dir=None, trace=False):
    """One step dict through the runner.  -> float32 CPU tensor [wanted, vocab] or None."""
    cache = runner.cache
    entries = []
    for e in step.get("entries", []):
        rid = e["id"]
        if rid not in cache.requests:
            cache.admit(rid)
        entries.append((rid, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
    logits = runner.step(entries) if entries else None
    result = traced = None
    if logits is not None:
        if trace:
            import torch

            from .. import ops
            pairs = torch.empty((logits.shape[0], 2), dtype=torch.int32, device=logits.device)
            ops.logit_trace(logits, pairs)
            traced = ops.read_logit_trace(pairs)
        result = logits.detach().float().cpu()
    runner.check()
    for rid in step.get("end", []):
        if rid in cache.requests:
            cache.release(rid)
    if result is not None and out_dir is not None:
        result.numpy().astype("<f4").tofile(os.path.join(out_dir, f"{step['step']}.f32"))
        if traced is not None:
            with open(os.path.join(out_dir, f"{step['step']}.lh.json"), "w") as fh:
                json.dump([[h, g] for h, g in traced], fh)
    return result


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the engine step by step "
                                 "and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    ap.add_argument("--max-tokens", required=True, type=int,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--trace", action="store_true",
                    help="also write <step>.lh.json: [hash of the logits, gap between the two largest] per wanted row")
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    print(f"trace_run: loading {a.model} ({a.dtype})", file=sys.stderr, flush=True)
    runner = make_runner(a.model, a.dtype, a.max_tokens, a.page_size)
    print("trace_run: ready", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        run_step(runner, step, a.out, trace=a.trace)
        print(f"done {step['step']}", flush=True)
    return 0
