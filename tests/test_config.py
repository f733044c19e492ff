"""Configuration and registry (no GPU)."""
import json

import pytest

from paged_batch_engine_b200.config import (ConfigError, Qwen2Config, get_architecture,
                                            known_architectures, load_config, register_architecture)
from tests.helpers import TINY_A, TINY_B, TINY_C


def test_reads_every_key_from_config_json():
    _, cfg = load_config(TINY_C)
    assert isinstance(cfg, Qwen2Config)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (88, 3, 6, 3)
    assert cfg.resolved_head_dim == 48 and cfg.intermediate_size == 208 and cfg.vocab_size == 517
    assert cfg.rope_theta == 50000.0 and cfg.rms_norm_eps == 3e-6 and not cfg.tie_word_embeddings
    assert [cfg.layer_window(i) for i in range(3)] == [None, 24, 24]
    assert cfg.eos_token_ids == (516,)
    _, b = load_config(TINY_B)
    assert b.eos_token_ids == (998, 999) and b.resolved_head_dim == 32


def test_model_spec_is_data_with_all_constants():
    _, cfg = load_config(TINY_C)
    spec = cfg.model_spec()
    assert len(spec.blocks) == 3 and [s.block for s in spec.run_order] == [0, 1, 2]
    a = spec.blocks[1].mixer.args
    assert a["num_heads"] == 6 and a["num_kv_heads"] == 3 and a["head_dim"] == 48 and a["window"] == 24
    assert a["qkv_bias"] is True and a["o_bias"] is False
    assert a["position"].args["theta"] == 50000.0 and a["position"].args["pairing"] == "half"
    assert spec.blocks[0].norm_mixer.args["eps"] == 3e-6
    assert spec.lm_head_name == "lm_head.weight"
    _, a_cfg = load_config(TINY_A)
    assert a_cfg.model_spec().lm_head_name is None          # tied


def test_folder_and_file_loading(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and cfg.vocab_size == 320
    _, cfg2 = load_config(str(tmp_path / "config.json"))
    assert cfg2.to_dict()["head_dim"] == 16


@pytest.mark.parametrize("change,needle", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(hidden_size=66), "head_dim"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size=0), "positive"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
])
def test_validation_errors(change, needle):
    d = dict(TINY_A)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        load_config(d)
    assert needle in str(e.value)


def test_missing_keys_and_unknown_architecture(tmp_path):
    d = dict(TINY_A)
    del d["intermediate_size"]
    with pytest.raises(ConfigError) as e:
        load_config(d)
    assert "intermediate_size" in str(e.value)
    d = dict(TINY_A, architectures=["NopeForCausalLM"])
    with pytest.raises(ConfigError) as e:
        load_config(d)
    assert "NopeForCausalLM" in str(e.value) and "Qwen2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))             # no config.json there
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_registry_accepts_another_architecture():
    class Other(Qwen2Config):
        pass
    register_architecture("OtherForCausalLM", Other, replace=True)
    assert "OtherForCausalLM" in known_architectures()
    _, cfg = load_config(dict(TINY_A, architectures=["OtherForCausalLM"]))
    assert isinstance(cfg, Other)
    with pytest.raises(ConfigError):
        register_architecture("OtherForCausalLM", Other)
    assert get_architecture("OtherForCausalLM").config_class is Other
