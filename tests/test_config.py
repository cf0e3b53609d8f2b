"""Configuration: typed values from the architecture's own keys, defaults, validation, and
the registry from architecture name to model."""
import json

import pytest

import tiny
from rllm_b200.config import (ConfigError, LlamaConfig, config_from_dict, load_config,
                              registered_architectures)


def test_llama_keys_and_defaults():
    arch, cfg = config_from_dict(tiny.TINY_B)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads,
            cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == \
        (96, 3, 3, 1, 32, 224, 384)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and not cfg.tie_word_embeddings
    rs = cfg.rope_scaling
    assert (rs.rope_type, rs.factor, rs.low_freq_factor, rs.high_freq_factor,
            rs.original_max_position_embeddings) == ("llama3", 8.0, 1.0, 4.0, 32)
    assert cfg.q_size == 96 and cfg.kv_size == 32


def test_head_dim_defaults_to_hidden_over_heads_and_kv_heads_to_heads():
    raw = {k: v for k, v in tiny.TINY_A.items() if k not in ("head_dim", "num_key_value_heads")}
    _, cfg = config_from_dict(raw)
    assert cfg.head_dim == 16 and cfg.num_key_value_heads == 4
    raw["head_dim"] = 0                      # the reference treats 0 as absent
    assert config_from_dict(raw)[1].head_dim == 16


def test_eps_aliases_and_theta_default():
    raw = dict(tiny.TINY_A)
    del raw["rms_norm_eps"], raw["rope_theta"]
    raw["norm_eps"] = 3e-6
    _, cfg = config_from_dict(raw)
    assert cfg.rms_norm_eps == 3e-6 and cfg.rope_theta == 10000.0


def test_model_type_alone_selects_the_architecture():
    raw = dict(tiny.TINY_A)
    del raw["architectures"]
    assert config_from_dict(raw)[0].name == "LlamaForCausalLM"


def test_unknown_architecture_lists_the_registered_ones():
    raw = dict(tiny.TINY_A, architectures=["MambaForCausalLM"], model_type="mamba")
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert "LlamaForCausalLM" in str(e.value) and "MambaForCausalLM" in str(e.value)
    assert "LlamaForCausalLM" in registered_architectures()


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "original_max_position_embeddings"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
])
def test_invalid_values_are_refused(patch, word):
    raw = dict(tiny.TINY_A)
    for k, v in patch.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_windows_per_layer():
    _, cfg = config_from_dict(tiny.TINY_C)
    assert [cfg.layer_window(i) for i in range(4)] == [24, None, 24, None]
    _, cfg = config_from_dict(dict(tiny.TINY_A, sliding_window=7))
    assert [cfg.layer_window(i) for i in range(2)] == [7, 7]


def test_round_trip_and_load_from_folder(tmp_path):
    _, cfg = config_from_dict(tiny.TINY_C)
    assert config_from_dict(cfg.to_dict())[1] == cfg
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_B))
    assert load_config(str(tmp_path))[1].vocab_size == 384
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_model_is_built_from_the_configuration_layer_by_layer():
    arch, cfg = config_from_dict(tiny.TINY_C)
    model = arch.build(cfg)
    assert len(model.blocks) == 4 and [c.block for c in model.schedule] == [0, 1, 2, 3]
    assert [b.mixer.window for b in model.blocks] == [24, None, 24, None]
    assert model.blocks[0].mixer.heads == 6 and model.blocks[0].mixer.kv_heads == 3
    assert model.blocks[0].ffn.intermediate == 176 and model.blocks[0].mixer_norm.eps == 3e-6
    assert model.head.tied_to is model.embedding
    specs = model.cache_specs()
    assert specs[0] == specs[2] != specs[1] == specs[3]


def test_special_token_ids():
    """bos_token_id / eos_token_id as config.json has them (a number or a list); a model that names
    none has none, whatever its vocabulary; ids beyond the vocabulary are refused; an explicit null
    survives the round trip."""
    from rllm_b200.config import config_from_dict
    base = dict(tiny.TINY_A)
    _, c = config_from_dict(base)
    assert c.bos_token_id is None and c.eos_token_ids == ()
    _, c = config_from_dict(dict(base, bos_token_id=1, eos_token_id=2))
    assert (c.bos_token_id, c.eos_token_ids) == (1, (2,))
    _, c = config_from_dict(dict(base, eos_token_id=[3, 250]))
    assert (c.bos_token_id, c.eos_token_ids) == (None, (3, 250))
    _, c3 = config_from_dict(dict(base, vocab_size=128256))
    assert (c3.bos_token_id, c3.eos_token_ids) == (None, ())
    _, again = config_from_dict(c.to_dict())
    assert again.eos_token_ids == (3, 250) and again.bos_token_id is None
    _, none = config_from_dict(dict(base, vocab_size=128256, bos_token_id=None, eos_token_id=None))
    assert none.bos_token_id is None and none.eos_token_ids == ()
    for bad in (dict(eos_token_id=256), dict(bos_token_id=-1), dict(eos_token_id="2"), dict(eos_token_id=[1, True])):
        with pytest.raises(ConfigError):
            config_from_dict(dict(base, **bad))


def test_special_token_ids_from_generation_config(tmp_path):
    """A folder whose config.json names no special ids takes them from generation_config.json
    beside it; config.json's own win."""
    import json
    from rllm_b200.config import load_config
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    (tmp_path / "generation_config.json").write_text(json.dumps({"bos_token_id": 5, "eos_token_id": [6, 7]}))
    _, c = load_config(str(tmp_path))
    assert (c.bos_token_id, c.eos_token_ids) == (5, (6, 7))
    (tmp_path / "config.json").write_text(json.dumps(dict(tiny.TINY_A, eos_token_id=9)))
    _, c = load_config(str(tmp_path))
    assert (c.bos_token_id, c.eos_token_ids) == (5, (9,))


def test_a_rope_rule_registered_from_outside_is_accepted_by_name():
    """`rope_scaling.rope_type` may be any registered rule: the configuration reader asks the
    registry, runs the rule's own check of its parameters, and keeps them for the rotary part."""
    from rllm_b200.config import config_from_dict
    from rllm_b200.parts import inverse_frequencies, register_rope_rule, registered_rope_rules

    def check(p):
        if p.get("every", 0) < 1:
            raise ValueError("rope_scaling.every must be >= 1")

    register_rope_rule("toy_every", lambda f, p: [x / p["factor"] if i % p["every"] == 0 else x for i, x in enumerate(f)], check)
    assert {"linear", "llama3", "toy_every"} <= set(registered_rope_rules())
    raw = dict(tiny.TINY_A, rope_scaling={"rope_type": "toy_every", "factor": 4.0, "every": 2})
    _, c = config_from_dict(raw)
    assert c.rope_scaling.rope_type == "toy_every" and c.rope_scaling.to_dict() == raw["rope_scaling"]
    _, again = config_from_dict(c.to_dict())
    assert again.rope_scaling == c.rope_scaling
    plain = inverse_frequencies(16, 10000.0)
    got = inverse_frequencies(16, 10000.0, c.rope_scaling)
    assert got == [x / 4.0 if i % 2 == 0 else x for i, x in enumerate(plain)]
    with pytest.raises(ConfigError, match="every"):
        config_from_dict(dict(tiny.TINY_A, rope_scaling={"rope_type": "toy_every", "factor": 4.0, "every": 0}))
    with pytest.raises(ConfigError, match="toy_every"):            # the refusal lists what is registered
        config_from_dict(dict(tiny.TINY_A, rope_scaling={"rope_type": "nonesuch", "factor": 2.0}))
