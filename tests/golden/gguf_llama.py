"""The reference's tiny GGUF-named llama fixtures, rebuilt from their seeds, with llama.cpp's own logits beside them.

mashbox-labs/mashbox tests its llama architecture against llama.cpp's CPU backend on tiny random GGUF files that it
does not commit: tools/gguf_fixtures/fixtures.py rebuilds each one from a seed (`write_dense`, fixtures.py:198-296;
cases at fixtures.py:433-458) and checks the file's sha256; what it commits are llama.cpp's logits for 16 prompt ids
and for 16 greedy steps after them (tests/fixtures/gguf/<name>.logits.f32, .greedy.json, .greedy.logits.f32; the bars
are tests/contracts/test_arch.py:11-38).  Four of them are this engine's architecture:

  llama-f32         rope_freqs.weight stored (random divisors in [1, 8)), q/k/v/o biases, GQA 8 over 2, own head
  llama-tied-f32    the same without output.weight (tied head)
  llama-eps-f32     rms eps 0.25, near the activations' mean square, so a norm that ignores the file's eps shows
  llama-linear-f32  linear rope scaling, factor 4, on top of the stored divisors

`tensors(name)` draws the same float32 tensors under the same GGUF names from the same seed in the same order as
fixtures.py does (q/k rows already in adjacent-pair order, as a GGUF file holds them); `config(name)` is the
config.json that says what the file's metadata says.  tests/golden/gguf_llama/ holds, copied from the reference
unchanged, llama.cpp's outputs, and tensors.sha256.json: the sha256 of every tensor as read back with gguf-py's
GGUFReader from the files that fixtures.py itself wrote here (their file sha256 equalled the committed ones), so the
tests know that `tensors()` rebuilds the reference's tensors bit for bit without needing gguf-py or the reference.

    python tests/golden/gguf_llama.py /path/to/mashbox        # writes tests/golden/gguf_llama/ again
"""
import hashlib
import json
import os

import numpy as np

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gguf_llama")
SIZES = dict(D=256, F=384, H=8, KV=2, HD=32, V=264, layers=4, theta=5e5, eps=1e-5)      # fixtures.py:191-192, vocab 45-55
CASES = {"llama-f32": dict(seed=10), "llama-tied-f32": dict(seed=40, tie=True), "llama-eps-f32": dict(seed=44, eps=0.25),
         "llama-linear-f32": dict(seed=43, linear=4.0)}                                   # fixtures.py:433, 448-452


def config(name):
    c, s = CASES[name], SIZES
    out = {"architectures": ["LlamaForCausalLM"], "hidden_act": "silu", "hidden_size": s["D"],
           "intermediate_size": s["F"], "num_attention_heads": s["H"], "num_key_value_heads": s["KV"],
           "head_dim": s["HD"], "num_hidden_layers": s["layers"], "vocab_size": s["V"], "rope_theta": s["theta"],
           "rms_norm_eps": c.get("eps", s["eps"]), "attention_bias": True, "tie_word_embeddings": bool(c.get("tie")),
           "max_position_embeddings": 4096}
    if c.get("linear"):
        out["rope_scaling"] = {"rope_type": "linear", "factor": c["linear"]}
    return out


def tensors(name):
    """-> {GGUF name: float32 array}, in the file's order"""
    c, s = CASES[name], SIZES
    D, F, H, KV, HD, V = s["D"], s["F"], s["H"], s["KV"], s["HD"], s["V"]
    rng = np.random.default_rng(c["seed"])
    f32 = lambda a: a.astype(np.float32)
    matrix = lambda rows, cols: f32(rng.standard_normal((rows, cols)) / np.sqrt(cols))
    norm = lambda n: f32(1.0 + 0.1 * rng.standard_normal(n))
    bias = lambda n: f32(0.2 * rng.standard_normal(n))
    out = {"token_embd.weight": f32(0.5 * rng.standard_normal((V, D))), "output_norm.weight": norm(D)}
    if not c.get("tie"):
        out["output.weight"] = matrix(V, D)
    out["rope_freqs.weight"] = f32(rng.uniform(1.0, 8.0, HD // 2))
    for layer in range(s["layers"]):
        p = f"blk.{layer}."
        out[p + "attn_norm.weight"] = norm(D)
        for role, rows, cols in (("attn_q", H * HD, D), ("attn_k", KV * HD, D), ("attn_v", KV * HD, D),
                                 ("attn_output", D, H * HD)):
            out[p + role + ".weight"] = matrix(rows, cols)
        for role, n in (("attn_q", H * HD), ("attn_k", KV * HD), ("attn_v", KV * HD), ("attn_output", D)):
            out[p + role + ".bias"] = bias(n)
        out[p + "ffn_norm.weight"] = norm(D)
        out[p + "ffn_gate.weight"] = matrix(F, D)
        out[p + "ffn_up.weight"] = matrix(F, D)
        out[p + "ffn_down.weight"] = matrix(D, F)
    return out


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a, dtype="<f4").tobytes()).hexdigest()


def reference(name):
    """-> dict(tokens, logits (16, V), greedy_ids, greedy_gaps, greedy_logits (16, V)): llama.cpp's outputs"""
    meta = json.load(open(os.path.join(HERE, name + ".json")))
    g = json.load(open(os.path.join(HERE, name + ".greedy.json")))
    V = meta["n_vocab"]
    return dict(tokens=meta["tokens"], logits=np.fromfile(os.path.join(HERE, name + ".logits.f32"), "<f4").reshape(-1, V),
                greedy_ids=g["ids"], greedy_gaps=g["gaps"],
                greedy_logits=np.fromfile(os.path.join(HERE, name + ".greedy.logits.f32"), "<f4").reshape(-1, V))


def tensor_digests():
    return json.load(open(os.path.join(HERE, "tensors.sha256.json")))


def main(reference_root):
    """Rebuilds the files with the reference's own tool, checks their sha256 against its committed ones, hashes the
    tensors as gguf-py reads them back, and copies llama.cpp's outputs."""
    import importlib.util
    import shutil
    import tempfile

    import gguf
    spec = importlib.util.spec_from_file_location(
        "ref_fixtures", os.path.join(reference_root, "tools", "gguf_fixtures", "fixtures.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    src = os.path.join(reference_root, "tests", "fixtures", "gguf")
    os.makedirs(HERE, exist_ok=True)
    digests = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name in CASES:
            path = tool.build(name, tmp)
            meta = json.load(open(os.path.join(src, name + ".json")))
            assert tool.sha256(path) == meta["gguf_sha256"], name
            digests[name] = {t.name: digest(np.asarray(t.data).reshape(-1)) for t in gguf.GGUFReader(path).tensors}
            for ext in (".json", ".logits.f32", ".greedy.json", ".greedy.logits.f32"):
                shutil.copyfile(os.path.join(src, name + ext), os.path.join(HERE, name + ext))
                os.chmod(os.path.join(HERE, name + ext), 0o644)
    json.dump(digests, open(os.path.join(HERE, "tensors.sha256.json"), "w"), indent=1, sort_keys=True)


if __name__ == "__main__":
    import sys
    main(sys.argv[1])
