"""Command line in the manner of `mashbox run` (src/mashbox/cli.py:1347-1427 of mashbox-labs/mashbox): the same
option names with the same meanings where this engine has the thing.

    python -m mashbox_b200 run <model-dir> --prompt TEXT | --prompt-ids 5,17,3
        [--thinking] [--max-tokens N] [--temperature T] [--top-p P] [--top-k K] [--seed N] [--ctx N] [--slots N]
        [--cache-dir DIR] [--no-warm] [--dtype bfloat16|float32] [--page-size N] [--chunk N] [--trace]
    python -m mashbox_b200 random <out-dir> --config config.json --seed N [--store bfloat16|float32]
    python -m mashbox_b200 env

Of the reference's `run` options, `--steps` (decode steps per device call) and `--no-kernels` (its plain JAX path) have
no counterpart: this engine always keeps two steps queued on the GPU, and its exact path is `--dtype float32`.

`--prompt TEXT` needs tokenizer.json in the model folder (and uses its chat template when tokenizer_config.json has
one); `--prompt-ids` needs none and prints ids.  Events go to stderr as JSON lines (`weights`, `loaded`, `warm`, `done`),
the answer to stdout.  A refusal prints one line and exits with 2.
"""
import argparse
import json
import os
import sys
import time

from .errors import MashboxError


def log(obj):
    print(obj if isinstance(obj, str) else json.dumps(obj), file=sys.stderr, flush=True)


def build_parser():
    ap = argparse.ArgumentParser(prog="mashbox_b200", description="A Llama-3 inference engine for one NVIDIA B200.")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("run", help="load a model folder and answer one prompt")
    p.add_argument("model", help="a model folder with config.json and safetensors weights")
    p.add_argument("--prompt", metavar="TEXT", help="answer one chat turn, print it and exit")
    p.add_argument("--prompt-ids", metavar="IDS", help="token ids separated by commas instead of text; prints ids")
    p.add_argument("--thinking", action="store_true", help="ask the chat template for the model's thinking mode")
    p.add_argument("--max-tokens", type=int, default=512, metavar="N", help="most new tokens")
    p.add_argument("--temperature", type=float, default=0.0, metavar="T", help="sampling temperature; 0 is greedy")
    p.add_argument("--top-p", type=float, default=1.0, metavar="P", help="nucleus sampling cut")
    p.add_argument("--top-k", type=int, default=0, metavar="K", help="top-k cut; 0 means none")
    p.add_argument("--seed", type=int, default=0, metavar="N", help="seed for sampled answers")
    p.add_argument("--ctx", default="auto", metavar="N|auto", help="context per request in tokens (prompt plus answer); "
                   "auto = the prompt plus --max-tokens")
    p.add_argument("--slots", type=int, default=1, metavar="N", help="requests decoded together")
    p.add_argument("--cache-dir", metavar="DIR", help="where compiled kernel libraries are kept (default: inside the "
                   "package when it can be written, else a per-user folder under the temporary directory)")
    p.add_argument("--no-warm", action="store_true", help="answer at once: without it a two-token answer is generated "
                   "first, so that compiling kernels and capturing graphs stay out of the reported times")
    p.add_argument("--trace", action="store_true", help="report per generated token the hash of its logits and the gap "
                   "between the two largest (also: MASHBOX_TRACE=1)")
    p.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"),
                   help="bfloat16: the serving kernels; float32: everything in true 32-bit")
    p.add_argument("--page-size", type=int, default=16, metavar="N", help="tokens per cache page")
    p.add_argument("--chunk", type=int, default=2048, metavar="N", help="most prompt tokens of a request in one step")
    r = sub.add_parser("random", help="write a model folder with seeded random weights")
    r.add_argument("out", help="folder to write config.json and model.safetensors to")
    r.add_argument("--config", required=True, help="a config.json of a supported architecture")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--store", default="bfloat16", choices=("bfloat16", "float32"))
    sub.add_parser("env", help="versions and GPU, for bug reports")
    return ap


def tokenizer_of(folder):
    path = os.path.join(folder, "tokenizer.json")
    if not os.path.isfile(path):
        raise MashboxError(f"--prompt needs {path}; give --prompt-ids instead")
    from tokenizers import Tokenizer
    return Tokenizer.from_file(path)


def chat_ids(folder, tok, text, thinking=False):
    """ids of one user turn: through the folder's chat template when it has one, else the bare text"""
    cfg = os.path.join(folder, "tokenizer_config.json")
    if os.path.isfile(cfg):
        tc = json.load(open(cfg))
        if tc.get("chat_template"):
            from jinja2.sandbox import ImmutableSandboxedEnvironment
            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
            text = env.from_string(tc["chat_template"]).render(
                messages=[dict(role="user", content=text)], add_generation_prompt=True, enable_thinking=bool(thinking),
                bos_token=tc.get("bos_token") or "", eos_token=tc.get("eos_token") or "")
            return tok.encode(text, add_special_tokens=False).ids
    return tok.encode(text).ids


def stop_ids_of(folder, cfg):
    ids = set()
    for src in (os.path.join(folder, "generation_config.json"),):
        if os.path.isfile(src):
            e = json.load(open(src)).get("eos_token_id")
            ids.update(e if isinstance(e, list) else [] if e is None else [e])
    e = cfg.get("eos_token_id")
    ids.update(e if isinstance(e, list) else [] if e is None else [e])
    return tuple(sorted(ids))


def cmd_run(a):
    from .engine.engine import Engine
    from .engine.loading import read_config_file
    if (a.prompt is None) == (a.prompt_ids is None):
        raise MashboxError("give --prompt TEXT or --prompt-ids IDS")
    t0 = time.time()
    if a.cache_dir:
        from .ops import build
        build.set_build_dir(a.cache_dir)
    cfg = read_config_file(a.model)
    tok = None
    if a.prompt is not None:
        tok = tokenizer_of(a.model)
        ids = chat_ids(a.model, tok, a.prompt, a.thinking)
        stops = stop_ids_of(a.model, cfg)
    else:
        try:
            ids = [int(x) for x in a.prompt_ids.split(",") if x.strip()]
        except ValueError:
            raise MashboxError("--prompt-ids takes integers separated by commas") from None
        stops = ()
    ctx = len(ids) + a.max_tokens if a.ctx == "auto" else int(str(a.ctx).lower().replace("k", "000"))
    ctx = -(-ctx // a.page_size) * a.page_size
    eng = Engine.from_folder(a.model, dtype=a.dtype, page_size=a.page_size, max_tokens=ctx * a.slots,
                             max_requests=a.slots, max_context=ctx, chunk=a.chunk,
                             max_tokens_per_step=a.chunk + a.slots, log=log, trace=True if a.trace else None)
    log(dict(event="loaded", seconds=round(time.time() - t0, 2), dtype=a.dtype, context=ctx, slots=a.slots))
    samp = None if a.temperature == 0 else [dict(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, seed=a.seed)]
    try:
        if not a.no_warm:
            t1 = time.time()
            eng.generate([ids], max_new=min(2, a.max_tokens), samp=samp)
            eng.generate([ids], max_new=min(2, a.max_tokens), samp=samp)      # shapes that came twice are graphs now
            log(dict(event="warm", seconds=round(time.time() - t1, 2)))
        r = eng.generate([ids], max_new=a.max_tokens, stop_ids=stops, samp=samp)
    except ValueError as e:
        raise MashboxError(str(e)) from None
    out = r["ids"][0]
    print(tok.decode(out) if tok is not None else ",".join(str(t) for t in out))
    t = r["timing"]
    done = dict(event="done", new_tokens=t["new_tokens"], prefill_s=round(t["prefill_s"], 3),
                decode_s=round(t["decode_s"], 3), finish=r["finish"][0])
    if "lh" in r:
        done["lh"] = r["lh"][0]
    log(done)
    return 0


def cmd_random(a):
    import torch
    from .config.registry import read_config
    from .weights.random_init import write_model_folder
    _, config = read_config(json.load(open(a.config)))
    write_model_folder(a.out, config, a.seed, dtype=getattr(torch, a.store))
    log(dict(event="written", folder=a.out, seed=a.seed, store=a.store))
    return 0


def cmd_env(a):
    import torch
    from . import __version__
    info = dict(mashbox_b200=__version__, torch=torch.__version__, cuda=torch.version.cuda,
                gpu=torch.cuda.get_device_name(0) if torch.cuda.is_available() else None)
    print(json.dumps(info))
    return 0


def main(argv=None):
    a = build_parser().parse_args(argv)
    try:
        return {"run": cmd_run, "random": cmd_random, "env": cmd_env}[a.cmd](a)
    except MashboxError as e:
        log(f"mashbox_b200: {e}")
        return 2
