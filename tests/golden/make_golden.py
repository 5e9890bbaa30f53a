"""Makes the golden files of this folder from mashbox-labs/mashbox's own test fixtures and importable functions.

The reference's model code (src/mashbox/gguf/archs/dense.py) needs JAX and cannot be imported on the machine this
was written on, so the plain implementation (tests/plain/llama.py) rests on the reference's formulas.  What the
reference does offer without JAX is used here as the anchor:

  * tests/fixtures/hf/llama and tests/fixtures/hf/mistral: tiny seeded models (config.json, model.safetensors) with
    the logits transformers computed for 16 tokens (logits.f32, meta.json).  They are copied as
    hf_llama.* / hf_mistral.* (config and tokens inside anchors.json).
  * mashbox.hf.adapter.llama3_factors / _llama_permute / gguf_name (numpy only): evaluated on a few inputs and
    stored in anchors.json, so that the tests compare value for value without the reference being present.

Run once:  python tests/golden/make_golden.py /path/to/mashbox   (the checkout that holds src/ and tests/).
It also prints the plain implementation's error against the transformers logits.
"""
import json
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref):
    sys.path.insert(0, os.path.join(ref, "src"))
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from mashbox.hf import adapter
    anchors = {"models": {}, "llama3_factors": [], "permute": [], "names": {}}
    for name in ("llama", "mistral"):
        d = os.path.join(ref, "tests", "fixtures", "hf", name)
        meta = json.load(open(os.path.join(d, "meta.json")))
        anchors["models"][name] = dict(config=json.load(open(os.path.join(d, "config.json"))), tokens=meta["tokens"],
                                       n_vocab=meta["n_vocab"], sha256=meta["sha256"])
        shutil.copyfile(os.path.join(d, "model.safetensors"), os.path.join(HERE, f"hf_{name}.safetensors"))
        shutil.copyfile(os.path.join(d, "logits.f32"), os.path.join(HERE, f"hf_{name}.logits.f32"))
        os.chmod(os.path.join(HERE, f"hf_{name}.safetensors"), 0o644)
        os.chmod(os.path.join(HERE, f"hf_{name}.logits.f32"), 0o644)
    for theta, dim, sc in ((500000.0, 16, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                original_max_position_embeddings=32)),
                           (500000.0, 32, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                               original_max_position_embeddings=64)),
                           (500000.0, 128, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                original_max_position_embeddings=8192)),
                           (500000.0, 64, dict(factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                               original_max_position_embeddings=8192)),
                           (10000.0, 48, dict(factor=3.0, low_freq_factor=2.0, high_freq_factor=5.0,
                                              original_max_position_embeddings=100))):
        f = adapter.llama3_factors(theta, dim, sc)
        anchors["llama3_factors"].append(dict(theta=theta, dim=dim, scaling=sc, factors=[float(x) for x in f]))
    for rows, heads in ((32, 2), (96, 6), (64, 1), (128, 4)):
        idx = adapter._llama_permute(np.arange(rows).reshape(rows, 1), heads)[:, 0]
        anchors["permute"].append(dict(rows=rows, heads=heads, index=[int(i) for i in idx]))
    for n in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight",
              "model.layers.3.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.bias",
              "model.layers.11.self_attn.v_proj.weight", "model.layers.2.self_attn.o_proj.weight",
              "model.layers.5.mlp.gate_proj.weight", "model.layers.5.mlp.up_proj.weight",
              "model.layers.5.mlp.down_proj.weight", "model.layers.7.input_layernorm.weight",
              "model.layers.7.post_attention_layernorm.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"):
        anchors["names"][n] = adapter.gguf_name("llama", n)
    json.dump(anchors, open(os.path.join(HERE, "anchors.json"), "w"), indent=1)

    from tests.plain import llama as plain
    for name in ("llama", "mistral"):
        m = anchors["models"][name]
        W = plain.read_safetensors(os.path.join(HERE, f"hf_{name}.safetensors"))
        got = plain.forward(m["config"], W, m["tokens"]).numpy()
        want = np.fromfile(os.path.join(HERE, f"hf_{name}.logits.f32"), np.float32).reshape(got.shape).astype(np.float64)
        nmse = float(((got - want) ** 2).sum() / (want ** 2).sum())
        print(name, "plain vs transformers logits: NMSE", nmse, "top-1 equal",
              int((got.argmax(-1) == want.argmax(-1)).sum()), "of", len(got))


if __name__ == "__main__":
    main(sys.argv[1])
