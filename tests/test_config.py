"""-m "not gpu": the typed configuration and the registry."""
import copy
import json
import os

import pytest

from mashbox_b200.config.llama import LlamaConfig, RopeScaling
from mashbox_b200.config.registry import ARCHITECTURES, architecture, read_config
from mashbox_b200.errors import ConfigError
from tests import helpers as H

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ANCHORS = json.load(open(os.path.join(GOLD, "anchors.json")))


def test_reads_the_reference_fixture_configs():
    c = LlamaConfig.from_hf(ANCHORS["models"]["llama"]["config"])
    assert (c.num_layers, c.hidden, c.num_heads, c.num_kv_heads, c.head_dim, c.intermediate, c.vocab) == \
        (3, 64, 4, 2, 16, 128, 256)
    assert c.rms_eps == 1e-6 and c.rope_theta == 500000.0 and c.attention_bias and not c.tie_embeddings
    assert c.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 32)
    m = LlamaConfig.from_hf(ANCHORS["models"]["mistral"]["config"])
    assert m.head_dim == 32 and m.hidden // m.num_heads == 16 and m.tie_embeddings and m.rope_scaling is None
    assert m.rope_theta == 1000000.0


def test_defaults():
    c = LlamaConfig.from_hf(dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, hidden_size=48,
                                 num_attention_heads=6, intermediate_size=100, vocab_size=77))
    assert c.num_kv_heads == 6 and c.head_dim == 8 and c.rms_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.rope_scaling is None and not c.tie_embeddings and not c.attention_bias
    c = LlamaConfig.from_hf(dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, hidden_size=48,
                                 num_attention_heads=6, intermediate_size=100, vocab_size=77, rope_theta=5e5,
                                 rope_scaling=dict(type="linear", factor=4.0)))
    assert c.rope_scaling == RopeScaling("linear", 4.0) and c.rope_theta == 5e5


@pytest.mark.parametrize("name", ["A", "B"])
def test_round_trip(name):
    cfg = H.TINY[name][0]
    entry, back = read_config(cfg.to_hf())
    assert back == cfg and entry is architecture("LlamaForCausalLM")


@pytest.mark.parametrize("change,word", [
    (dict(hidden_act="gelu"), "hidden_act"), (dict(quantization_config=dict(quant_method="awq")), "quantization_config"),
    (dict(mlp_bias=True), "mlp_bias"), (dict(sliding_window=4096), "sliding_window"),
    (dict(use_sliding_window=True), "use_sliding_window"), (dict(layer_types=["sliding_attention"]), "layer_types"),
    (dict(num_local_experts=8), "num_local_experts"), (dict(rope_scaling=dict(rope_type="yarn", factor=2)), "rope type"),
    (dict(num_key_value_heads=3), "num_key_value_heads"), (dict(architectures=[]), "architectures"),
    (dict(architectures=["GPT2LMHeadModel"]), "GPT2LMHeadModel"), (dict(hidden_size=None), "hidden_size")])
def test_refusals_name_the_field(change, word):
    cfg = copy.deepcopy(H.TINY_A.to_hf())
    cfg.update(change)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert word in str(e.value) and "\n" not in str(e.value)


def test_both_reference_names_are_registered():
    architecture("LlamaForCausalLM")
    assert {"LlamaForCausalLM", "MistralForCausalLM"} <= set(ARCHITECTURES)


def test_model_spec_is_data():
    from mashbox_b200.models.llama import model_spec
    spec = model_spec(H.TINY_B)
    assert len(spec.layers) == 3 and [r.layer for r in spec.schedule] == [0, 1, 2]
    assert all(r.cache == r.layer and r.write for r in spec.schedule)
    b = spec.layers[1].block
    assert b.kind == "prenorm" and b.params["norm"].params["eps"] == 1e-6
    m = b.params["mixer"]
    assert m.kind == "attention" and m.params["heads"] == 6 and m.params["kv_heads"] == 1 and m.params["head_dim"] == 32
    assert m.params["position"].kind == "rope" and b.params["ffn"].params["intermediate"] == 320
