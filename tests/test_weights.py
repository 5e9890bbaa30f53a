"""-m "not gpu": reading weights by name, the one error that lists what does not fit, random-weights mode."""
import json
import os

import numpy as np
import pytest
import torch

from mashbox_b200.config.registry import read_config
from mashbox_b200.engine.loading import build_model, read_config_file
from mashbox_b200.errors import WeightError
from mashbox_b200.models.llama import permute_rows
from mashbox_b200.weights.random_init import random_tensors, write_model_folder
from mashbox_b200.weights.safetensors_io import DictSource, SafetensorsSource, write_safetensors
from tests import helpers as H
from tests.plain import llama as plain

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ANCHORS = json.load(open(os.path.join(GOLD, "anchors.json")))


def stored(name="A", dtype=torch.float32):
    cfg = H.TINY[name][0]
    entry, _ = read_config(cfg.to_hf())
    return cfg, random_tensors(entry.stored_tensors(cfg), 3, dtype=dtype)


def build(cfg, tensors, dtype="float32"):
    return build_model(cfg.to_hf(), DictSource(tensors), dtype, "cpu")


def test_folder_round_trip_and_dtypes(tmp_path):
    d = write_model_folder(str(tmp_path / "m"), H.TINY_B, 1, dtype=torch.bfloat16)
    src = SafetensorsSource(d)
    cfg, want = stored("B", torch.bfloat16)
    want = random_tensors(read_config(cfg.to_hf())[0].stored_tensors(cfg), 1, dtype=torch.bfloat16)
    assert sorted(src.names()) == sorted(want)
    for n in want:
        assert src.info(n) == (torch.bfloat16, tuple(want[n].shape))
        assert torch.equal(src.get(n), want[n])
    # the plain implementation's own reader sees the same values
    W = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    assert torch.equal(W["model.layers.2.mlp.up_proj.weight"], want["model.layers.2.mlp.up_proj.weight"].double())
    model = build_model(read_config_file(d), src, "bfloat16", "cpu")
    blk = model.layers[0]
    assert blk.mixer.wqkv.dtype == torch.bfloat16 and blk.ffn.wgu.dtype == torch.bfloat16      # matrices: compute dtype
    assert blk.norm1.weight.dtype == torch.float32 and blk.mixer.bqkv.dtype == torch.float32    # vectors: float32
    model32 = build_model(read_config_file(d), src, "float32", "cpu")
    assert model32.layers[0].mixer.wqkv.dtype == torch.float32
    assert torch.equal(model32.layers[0].mixer.wqkv, blk.mixer.wqkv.float())                    # bf16 -> f32 is exact


def test_seed_and_name_decide_the_values():
    cfg, a = stored()
    _, b = stored()
    assert all(torch.equal(a[n], b[n]) for n in a)
    entry, _ = read_config(cfg.to_hf())
    c = random_tensors(entry.stored_tensors(cfg), 4)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    one = random_tensors({"model.norm.weight": entry.stored_tensors(cfg)["model.norm.weight"]}, 3)
    assert torch.equal(one["model.norm.weight"], a["model.norm.weight"])         # independent of the other tensors


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    cfg, t = stored("B")
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.layers.0.self_attn.k_proj.bias"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)          # knowingly skipped, not an error
    t["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)                   # a layer the model does not have
    t["model.some_adapter.weight"] = torch.zeros(2, 2)
    t["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(10, 96)
    t["model.norm.weight"] = torch.zeros(97)
    with pytest.raises(WeightError) as e:
        build(cfg, t)
    msg = str(e.value)
    assert "\n" not in msg
    for word in ("missing:", "blk.1.ffn_up.weight", "blk.0.attn_k.bias", "unexpected:", "model.layers.7.mlp.up_proj.weight",
                 "model.some_adapter.weight", "wrong shape:", "model.layers.2.self_attn.q_proj.weight is [10, 96]",
                 "[192, 96]", "model.norm.weight is [97]"):
        assert word in msg, word
    assert "inv_freq" not in msg


def test_tied_model_drops_a_stored_head_and_untied_needs_it():
    cfg, t = stored("A")
    t["lm_head.weight"] = torch.zeros(256, 64)
    m = build(cfg, t)
    assert m.head.weight is m.embedding.table
    cfgb, tb = stored("B")
    del tb["lm_head.weight"]
    with pytest.raises(WeightError, match="missing: output.weight"):
        build(cfgb, tb)


def test_hugging_face_q_and_k_rows_are_permuted_and_gguf_names_are_not():
    cfg, t = stored("B")
    m = build(cfg, t)
    H_, KV, HD = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    wq = t["model.layers.1.self_attn.q_proj.weight"]
    assert torch.equal(m.layers[1].mixer.wqkv[:H_ * HD], plain.permute_rows(wq, H_))
    assert torch.equal(m.layers[1].mixer.wqkv[H_ * HD:(H_ + KV) * HD],
                       plain.permute_rows(t["model.layers.1.self_attn.k_proj.weight"], KV))
    assert torch.equal(m.layers[1].mixer.bqkv[:H_ * HD], plain.permute_rows(t["model.layers.1.self_attn.q_proj.bias"], H_))
    assert torch.equal(m.layers[1].mixer.wqkv[(H_ + KV) * HD:], t["model.layers.1.self_attn.v_proj.weight"])
    for case in ANCHORS["permute"]:
        idx = permute_rows(torch.arange(case["rows"]).reshape(-1, 1), case["heads"])[:, 0]
        assert idx.tolist() == case["index"]
    # the same model under the GGUF names of the reference's dense module, rows already permuted, factors as a tensor
    from mashbox_b200.parts.position import llama3_factors
    g = {}
    for hf, gg in ANCHORS["names"].items():
        if gg is None:
            continue
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    role = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
            "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
            "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm"}
    for n, x in t.items():
        if n in names:
            g[names[n]] = x
            continue
        p = n.split(".")
        r = role[".".join(p[3:-1])]
        if r == "attn_q":
            x = plain.permute_rows(x, H_)
        elif r == "attn_k":
            x = plain.permute_rows(x, KV)
        g[f"blk.{p[2]}.{r}.{p[-1]}"] = x
    s = cfg.rope_scaling
    g["rope_freqs.weight"] = torch.from_numpy(llama3_factors(cfg.rope_theta, HD, s.factor, s.low_freq_factor,
                                                            s.high_freq_factor, s.original_max_position))
    m2 = build(cfg, g)
    assert torch.equal(m2.layers[1].mixer.wqkv, m.layers[1].mixer.wqkv)
    assert torch.equal(m2.layers[2].ffn.wgu, m.layers[2].ffn.wgu)
    assert torch.equal(m2.layers[0].mixer.position.freqs, m.layers[0].mixer.position.freqs)


def test_name_map_equals_the_reference():
    from mashbox_b200.models.llama import canonical_names
    import dataclasses
    cfg = dataclasses.replace(H.TINY_B, num_layers=12)
    canon = canonical_names(cfg)
    for hf, gg in ANCHORS["names"].items():
        got = canon(hf)
        assert (None if got is None else got[0]) == gg, hf


def test_frequency_table_equals_the_reference_factors():
    from mashbox_b200.parts.position import RotaryEncoding, base_frequencies, llama3_factors
    for case in ANCHORS["llama3_factors"]:
        sc = case["scaling"]
        got = llama3_factors(case["theta"], case["dim"], sc["factor"], sc["low_freq_factor"], sc["high_freq_factor"],
                             sc["original_max_position_embeddings"])
        assert np.array_equal(got, np.asarray(case["factors"], np.float32))
        r = RotaryEncoding(case["dim"], case["dim"], case["theta"],
                           ("llama3", sc["factor"], sc["low_freq_factor"], sc["high_freq_factor"],
                            sc["original_max_position_embeddings"]))
        assert np.array_equal(r.frequencies(), plain.rope_frequencies(case["theta"], case["dim"], dict(sc, rope_type="llama3")))
    lin = RotaryEncoding(32, 32, 1e4, ("linear", 4.0)).frequencies()
    assert np.array_equal(lin, plain.rope_frequencies(1e4, 32, dict(rope_type="linear", factor=4.0)))
    assert np.array_equal(RotaryEncoding(32, 32, 1e4).frequencies(), base_frequencies(1e4, 32))


def test_bad_files(tmp_path):
    d = tmp_path / "empty"
    d.mkdir()
    with pytest.raises(WeightError, match="no safetensors weights"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="no safetensors header .the file is 2 bytes"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes((10 ** 12).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError, match="announce a header of 1000000000000"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes((6).to_bytes(8, "little") + b"{nope}")
    with pytest.raises(WeightError, match="header is not JSON"):
        SafetensorsSource(str(d))
    write_safetensors(str(d / "model.safetensors"), {"a": torch.zeros(3, dtype=torch.float32)})
    raw = bytearray((d / "model.safetensors").read_bytes())
    (d / "model.safetensors").write_bytes(bytes(raw).replace(b'"F32"', b'"F8X"'))
    with pytest.raises(WeightError, match="tensor a has dtype F8X"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes(bytes(raw)[:-4])
    with pytest.raises(WeightError, match=r"tensor a of shape \[3\] and dtype F32 needs 12 bytes, its entry gives bytes 0..12 of 8"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes(bytes(raw))
    # a second copy of the weights under another name is not read (nor a tensor taken twice)
    write_safetensors(str(d / "consolidated.safetensors"), {"a": torch.ones(3, dtype=torch.float32)})
    src = SafetensorsSource(str(d))
    assert src.names() == ["a"] and float(src.get("a").sum()) == 0.0
    (d / "model.safetensors").unlink()
    assert float(SafetensorsSource(str(d)).get("a").sum()) == 3.0            # ... unless it is all there is
    write_safetensors(str(d / "other.safetensors"), {"a": torch.ones(3, dtype=torch.float32)})
    with pytest.raises(WeightError, match="tensor a is in consolidated.safetensors and in other.safetensors"):
        SafetensorsSource(str(d))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "model-00001-of-00002.safetensors"}}))
    with pytest.raises(WeightError, match="names model-00001-of-00002.safetensors, which the folder does not have"):
        SafetensorsSource(str(d))


def test_reads_the_reference_fixture_files():
    """the loader binds the reference's two Hugging Face fixtures as the plain implementation reads them: q/k rows and
    biases permuted for adjacent pairs, q|k|v stacked, the llama3 divisors from rope_parameters, the tied head"""
    for name in ("llama", "mistral"):
        m = ANCHORS["models"][name]
        c = plain.sizes(m["config"])
        W = plain.read_safetensors(os.path.join(GOLD, f"hf_{name}.safetensors"))
        model = build_model(m["config"], DictSource({k: v.float() for k, v in W.items()}), "float32", "cpu")
        assert len(model.layers) == c["L"]
        for l, block in enumerate(model.layers):
            p = f"model.layers.{l}.self_attn."
            want = torch.cat([plain.permute_rows(W[p + "q_proj.weight"], c["H"]),
                              plain.permute_rows(W[p + "k_proj.weight"], c["KV"]), W[p + "v_proj.weight"]]).float()
            assert torch.equal(block.mixer.wqkv, want)
            if p + "q_proj.bias" in W:
                wb = torch.cat([plain.permute_rows(W[p + "q_proj.bias"], c["H"]),
                                plain.permute_rows(W[p + "k_proj.bias"], c["KV"]), W[p + "v_proj.bias"]]).float()
                assert torch.equal(block.mixer.bqkv, wb)
            assert np.array_equal(block.mixer.position.freqs.numpy(),
                                  plain.rope_frequencies(c["theta"], c["HD"], c["scaling"]))
        tied = c["tie"]
        assert (model.head.weight.data_ptr() == model.embedding.table.data_ptr()) == tied


def test_stored_divisors_and_the_linear_factor_apply_together():
    """a GGUF-named file may bring rope_freqs.weight AND ask for linear scaling: angle = pos * inv / divisor / factor
    (src/mashbox/gguf/archs/dense.py:93-94, 316-317)"""
    from mashbox_b200.parts.position import RotaryEncoding, base_frequencies
    div = np.linspace(1.0, 8.0, 16).astype(np.float32)
    got = RotaryEncoding(32, 32, 5e5, ("linear", 4.0)).frequencies(div)
    want = ((base_frequencies(5e5, 32) / div).astype(np.float32) * np.float32(0.25)).astype(np.float32)
    assert np.array_equal(got, want)
    assert np.array_equal(got, plain.rope_frequencies(5e5, 32, dict(rope_type="linear", factor=4.0), div))
    # stored divisors stand in for the llama3 ones the configuration would give
    sc = ("llama3", 8.0, 1.0, 4.0, 64)
    assert np.array_equal(RotaryEncoding(32, 32, 5e5, sc).frequencies(div), (base_frequencies(5e5, 32) / div).astype(np.float32))
