"""-m gpu: the ENGINE (loader, step function, cache, kernels) on the reference's own fixtures, against logits that neither
this repository nor its plain implementation produced.

  * tests/golden/hf_llama, hf_mistral: mashbox-labs/mashbox's committed Hugging Face fixtures with transformers' float32
    logits (tests/fixtures/hf/{llama,mistral}; its own engine is held to NMSE <= 1e-4 on them, whole and as a prefill
    of 8 followed by 8 one-token steps, tests/cpu/test_hf_safetensors.py:42, 100-112).  llama: q/k/v/o biases, llama3
    scaling through rope_parameters, own head; mistral: head_dim != hidden / heads, tied head.
  * tests/golden/gguf_llama: its four GGUF-named llama fixtures with llama.cpp's logits and greedy ids
    (tests/contracts/test_arch.py:11-38, 307-409): stored rope_freqs, rows already in adjacent-pair order, a tied head,
    eps 0.25, linear scaling.

Bars.  float32: NMSE <= 1e-10 (the reference's bar between two float32 programs is 1e-4).  bfloat16: the weights are
rounded to bfloat16 at load, so the measure of what bfloat16 costs here is the plain implementation with the same
rounded weights and bfloat16 storage against the fixture's logits; the engine may be at most twice that far away.
"""
import json
import os
import shutil

import numpy as np
import pytest
import torch

from tests.golden import gguf_llama
from tests.plain import llama as plain
from tests.tolerances import BF16_NOISE_FACTOR, NMSE_F32, nmse

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
ANCHORS = json.load(open(os.path.join(GOLD, "anchors.json")))
DEV = "cuda:0"
SPLIT = 8
NEAR_TIE_GAP = 0.5          # tests/contracts/test_arch.py, bar 3


def runner_for(cfg, tensors, dtype, page_size=16, options=None):
    from mashbox_b200 import ops
    from mashbox_b200.config.engine import EngineConfig
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.engine.runner import ModelRunner
    from mashbox_b200.weights.safetensors_io import DictSource
    model = build_model(cfg, DictSource(tensors), dtype, DEV, ops=ops)
    ecfg = EngineConfig(dtype=dtype, page_size=page_size, max_tokens=128, max_requests=2, max_tokens_per_step=64,
                        chunk=64, device=DEV)
    return model, ModelRunner(model, ecfg, options)


def all_logits(runner, tokens, split=None):
    """logits at every position: one step, or `split` tokens in one step and the rest one by one"""
    from mashbox_b200.engine.replay import run_step
    n = len(tokens) if split is None else split
    steps = [dict(entries=[dict(id="a", tokens=tokens[:n], want=list(range(n)))], end=[])]
    steps += [dict(entries=[dict(id="a", tokens=[t], want=[0])], end=[]) for t in tokens[n:]]
    steps[-1]["end"] = ["a"]
    out = [run_step(runner, dict(s, step=i)).numpy() for i, s in enumerate(steps)]
    runner.cache.check()
    return np.concatenate(out)


def bf16_noise(cfg, tensors, tokens, want):
    """how far bfloat16 weights and bfloat16 storage put the plain model from the fixture's logits"""
    rounded = {k: (plain.round_bf16(v) if v.dim() == 2 else v) for k, v in tensors.items()}
    return nmse(plain.forward(cfg, rounded, tokens, held=plain.round_bf16).numpy(), want)


def compare(cfg, tensors, tokens, want, dtype, page_size, what):
    _, runner = runner_for(cfg, tensors, dtype, page_size)
    for split in (None, SPLIT):
        got = all_logits(runner, tokens, split)
        assert got.shape == want.shape and np.isfinite(got).all()
        e = nmse(got, want)
        cut = "whole" if split is None else f"{split} + {len(tokens) - split} one by one"
        if dtype == "float32":
            assert e <= NMSE_F32, f"{what}, {cut}: float32 NMSE {e:.3e}"
            assert (got.argmax(-1) == want.argmax(-1)).all()
        else:
            noise = bf16_noise(cfg, tensors, tokens, want)
            assert 0 < noise < 1e-3
            assert e <= BF16_NOISE_FACTOR * noise, f"{what}, {cut}: bfloat16 NMSE {e:.3e}, its own noise {noise:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["llama", "mistral"])
def test_engine_matches_transformers_logits(name, dtype):
    m = ANCHORS["models"][name]
    W = {k: v.float() for k, v in plain.read_safetensors(os.path.join(GOLD, f"hf_{name}.safetensors")).items()}
    want = np.fromfile(os.path.join(GOLD, f"hf_{name}.logits.f32"), np.float32).reshape(len(m["tokens"]), -1)
    compare(m["config"], W, m["tokens"], want, dtype, 8 if name == "llama" else 16, f"hf {name}")


@pytest.mark.parametrize("name", ["llama", "mistral"])
def test_engine_reads_the_fixture_folder_itself(tmp_path, name):
    """the same through the loader's own safetensors reader and the folder entry point"""
    from mashbox_b200.engine.replay import make_runner
    m = ANCHORS["models"][name]
    d = tmp_path / name
    d.mkdir()
    (d / "config.json").write_text(json.dumps(m["config"]))
    shutil.copyfile(os.path.join(GOLD, f"hf_{name}.safetensors"), d / "model.safetensors")
    runner = make_runner(str(d), "float32", 64, page_size=8)
    want = np.fromfile(os.path.join(GOLD, f"hf_{name}.logits.f32"), np.float32).reshape(len(m["tokens"]), -1)
    assert nmse(all_logits(runner, m["tokens"]), want) <= NMSE_F32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(gguf_llama.CASES))
def test_engine_matches_llama_cpp_logits(name, dtype):
    cfg = gguf_llama.config(name)
    W = {k: torch.from_numpy(v) for k, v in gguf_llama.tensors(name).items()}
    ref = gguf_llama.reference(name)
    compare(cfg, W, ref["tokens"], ref["logits"], dtype, 8, name)


@pytest.mark.parametrize("name", list(gguf_llama.CASES))
def test_engine_greedy_ids_match_llama_cpp(name):
    """16 greedy ids after the 16 prompt ids through generate(): all equal llama.cpp's, or the first difference is at
    a step where llama.cpp's own top-two gap is under 0.5 logit."""
    from mashbox_b200 import ops
    from mashbox_b200.config.engine import EngineConfig
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.weights.safetensors_io import DictSource
    cfg = gguf_llama.config(name)
    W = {k: torch.from_numpy(v) for k, v in gguf_llama.tensors(name).items()}
    ref = gguf_llama.reference(name)
    model = build_model(cfg, DictSource(W), "float32", DEV, ops=ops)
    eng = Engine(model, EngineConfig(dtype="float32", page_size=8, max_tokens=128, max_requests=2,
                                     max_tokens_per_step=64, chunk=64, device=DEV))
    ids = eng.generate([ref["tokens"]], max_new=len(ref["greedy_ids"]))["ids"][0]
    diff = [i for i, (a, b) in enumerate(zip(ids, ref["greedy_ids"])) if a != b]
    assert not diff or ref["greedy_gaps"][diff[0]] < NEAR_TIE_GAP, (ids, ref["greedy_ids"])
    near = [i for i, g in enumerate(ref["greedy_gaps"]) if g < NEAR_TIE_GAP]
    stable = near[0] if near else len(ids)
    assert ids[:stable] == ref["greedy_ids"][:stable]
