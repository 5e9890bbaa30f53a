"""-m "not gpu": the plain implementation against what mashbox-labs/mashbox offers without JAX: transformers' logits of
its two committed Hugging Face fixtures, and its numpy-only helpers evaluated once (tests/golden/anchors.json)."""
import json
import os

import numpy as np
import pytest
import torch

from tests.plain import llama as plain

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ANCHORS = json.load(open(os.path.join(GOLD, "anchors.json")))


@pytest.mark.parametrize("name", ["llama", "mistral"])
def test_plain_matches_transformers_logits(name):
    m = ANCHORS["models"][name]
    W = plain.read_safetensors(os.path.join(GOLD, f"hf_{name}.safetensors"))
    got = plain.forward(m["config"], W, m["tokens"]).numpy()
    want = np.fromfile(os.path.join(GOLD, f"hf_{name}.logits.f32"), np.float32).reshape(got.shape).astype(np.float64)
    nmse = ((got - want) ** 2).sum() / (want ** 2).sum()
    assert nmse <= 1e-10                      # the reference's own bar is 1e-4 (tests/cpu/test_hf_safetensors.py:42)
    assert (got.argmax(-1) == want.argmax(-1)).all()


def test_llama3_factors_equal_the_reference():
    for case in ANCHORS["llama3_factors"]:
        got = plain.llama3_factors(case["theta"], case["dim"], case["scaling"])
        assert np.array_equal(got, np.asarray(case["factors"], np.float32))


def test_permutation_equals_the_reference():
    for case in ANCHORS["permute"]:
        idx = plain.permute_rows(torch.arange(case["rows"]).reshape(-1, 1), case["heads"])[:, 0]
        assert idx.tolist() == case["index"]


def test_adjacent_rotation_on_permuted_rows_equals_halves_rotation():
    torch.manual_seed(0)
    T, H, HD = 5, 3, 8
    x = torch.randn(T, H * HD, dtype=torch.float64)
    freqs = plain.rope_frequencies(10000.0, HD, None)
    pos = np.arange(T) + 3
    halves = plain.rope_halves(x.reshape(T, H, HD), pos, freqs).reshape(T, H * HD)
    perm = plain.permute_rows(torch.arange(H * HD).reshape(-1, 1), H)[:, 0]
    adjacent = plain.rope_adjacent(x[:, perm].reshape(T, H, HD), pos, freqs).reshape(T, H * HD)
    assert torch.allclose(adjacent, halves[:, perm], atol=1e-14)


def test_attention_window_and_causality():
    torch.manual_seed(1)
    T, H, KV, HD = 9, 4, 2, 8
    q, k, v = torch.randn(T, H, HD, dtype=torch.float64), torch.randn(T, KV, HD, dtype=torch.float64), \
        torch.randn(T, KV, HD, dtype=torch.float64)
    full = plain.attention(q, k, v, HD ** -0.5)
    # changing a later key or value never changes an earlier query's output
    k2, v2 = k.clone(), v.clone()
    k2[6:] += 1.0
    v2[6:] -= 2.0
    assert torch.equal(plain.attention(q, k2, v2, HD ** -0.5)[:6], full[:6])
    # window 1 = each query sees itself only
    w1 = plain.attention(q, k, v, HD ** -0.5, window=1)
    want = v.repeat_interleave(H // KV, 1).reshape(T, H * HD)
    assert torch.allclose(w1, want, atol=1e-14)
    # a window as long as the sequence changes nothing
    assert torch.allclose(plain.attention(q, k, v, HD ** -0.5, window=T), full, atol=1e-14)


def test_rounded_model_is_close_to_the_exact_one():
    m = ANCHORS["models"]["llama"]
    W = plain.read_safetensors(os.path.join(GOLD, "hf_llama.safetensors"))
    a = plain.forward(m["config"], W, m["tokens"]).numpy()
    b = plain.forward(m["config"], W, m["tokens"], held=plain.round_bf16).numpy()
    e = ((a - b) ** 2).sum() / (a ** 2).sum()
    assert 0 < e < 1e-3


# ---------------------------------------------------------------------------------------- llama.cpp's logits (GGUF names)
from tests.golden import gguf_llama

LLAMA_CPP_NMSE = 1e-10      # the reference's bar between two float32 programs is 1e-4 (tests/contracts/test_arch.py:11-38)


def gguf_case(name):
    return gguf_llama.config(name), {k: torch.from_numpy(v) for k, v in gguf_llama.tensors(name).items()}, \
        gguf_llama.reference(name)


@pytest.mark.parametrize("name", list(gguf_llama.CASES))
def test_rebuilt_gguf_tensors_are_the_reference_files_tensors(name):
    want = gguf_llama.tensor_digests()[name]
    got = {k: gguf_llama.digest(v) for k, v in gguf_llama.tensors(name).items()}
    assert got == want


@pytest.mark.parametrize("name", list(gguf_llama.CASES))
def test_plain_matches_llama_cpp_logits(name):
    """GGUF-named tensors: q/k rows already in adjacent-pair order, rope_freqs.weight as stored, biases, a tied head,
    an eps near the activations' mean square, linear scaling on top of the stored divisors."""
    cfg, W, ref = gguf_case(name)
    got = plain.forward(cfg, W, ref["tokens"]).numpy()
    from tests.tolerances import nmse
    assert nmse(got, ref["logits"]) <= LLAMA_CPP_NMSE
    assert (got.argmax(-1) == ref["logits"].argmax(-1)).all()


def test_the_gguf_fixtures_show_what_they_are_for():
    """Each option the fixtures pin moves the logits far beyond the bar when it is ignored: the stored divisors, the
    linear factor, the eps of the file, the pre-permuted row order."""
    from tests.tolerances import nmse
    cfg, W, ref = gguf_case("llama-linear-f32")
    no_factor = dict(cfg, rope_scaling=None)
    assert nmse(plain.forward(no_factor, W, ref["tokens"]).numpy(), ref["logits"]) > 1e-3
    no_divisors = {k: v for k, v in W.items() if k != "rope_freqs.weight"}
    assert nmse(plain.forward(cfg, no_divisors, ref["tokens"]).numpy(), ref["logits"]) > 1e-3
    cfg, W, ref = gguf_case("llama-eps-f32")
    assert nmse(plain.forward(dict(cfg, rms_norm_eps=1e-5), W, ref["tokens"]).numpy(), ref["logits"]) > 1e-3
    cfg, W, ref = gguf_case("llama-f32")
    again = dict(W)
    again["blk.0.attn_q.weight"] = plain.permute_rows(W["blk.0.attn_q.weight"], cfg["num_attention_heads"])
    assert nmse(plain.forward(cfg, again, ref["tokens"]).numpy(), ref["logits"]) > 1e-3
