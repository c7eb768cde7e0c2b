import json

import pytest

from forge_b200.config import (ConfigError, LlamaConfig, config_from_dict, load_config, register_architecture,
                               registered_architectures, unregister_architecture)
from helpers import TINY


def test_reads_every_key_and_defaults():
    c = config_from_dict(TINY["B"])
    assert isinstance(c, LlamaConfig)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (387, 96, 264, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and c.attention_bias and c.tie_word_embeddings
    d = dict(TINY["A"])
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "max_position_embeddings",
              "tie_word_embeddings", "attention_bias"):
        d.pop(k)
    c = config_from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads == 4 and c.head_dim == 16
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6 and c.max_position_embeddings == 4096
    assert not c.tie_word_embeddings and not c.attention_bias


def test_qwen2_name_defaults_to_bias():
    d = dict(TINY["A"], architectures=["Qwen2ForCausalLM"])
    d.pop("attention_bias")
    assert config_from_dict(d).attention_bias is True


@pytest.mark.parametrize("patch,needle", [
    ({"architectures": ["FalconForCausalLM"]}, "no model registered"),
    ({"architectures": []}, "architectures"),
    ({"vocab_size": None}, "vocab_size"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"head_dim": 15}, "even"),
    ({"num_hidden_layers": 0}, "positive"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rms_norm_eps": 0.0}, "positive"),
])
def test_bad_configs_are_refused(patch, needle):
    d = dict(TINY["A"], **patch)
    with pytest.raises(ConfigError, match=needle):
        config_from_dict(d)


def test_round_trip_and_load(tmp_path):
    c = config_from_dict(TINY["A"])
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nope"))


def test_plan_is_data():
    plan = config_from_dict(TINY["B"]).plan()
    assert plan.schedule == [0, 1, 2] and len(plan.layers) == 3
    l0 = plan.layers[0]
    assert l0.block == "pre_norm" and l0.mixer.kind == "attention" and l0.feed_forward.kind == "swiglu"
    assert l0.mixer.params["position"].kind == "rope" and l0.mixer.params["position"].params["theta"] == 500000.0
    assert l0.norms["input"].params["eps"] == 1e-6 and l0.weight_prefix == "model.layers.0."
    assert plan.lm_head.params["tied"] is True


def test_registry_takes_new_architectures():
    class Toy:
        @classmethod
        def from_dict(cls, d, architecture):
            return cls()

        def plan(self):
            return None

        def to_dict(self):
            return {}
    register_architecture("ToyForCausalLM", Toy)
    try:
        assert "ToyForCausalLM" in registered_architectures()
        assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), Toy)
        with pytest.raises(ConfigError, match="already registered"):
            register_architecture("ToyForCausalLM", Toy)
    finally:
        unregister_architecture("ToyForCausalLM")
