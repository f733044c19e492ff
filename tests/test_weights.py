"""Weight loading by tensor name, its one error, and the random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from paged_batch_engine_b200.config import load_config
from paged_batch_engine_b200.engine.runner import build_model
from paged_batch_engine_b200.weights import (ParamSpec, SafetensorsFile, WeightsError, load_weights,
                                             save_file, write_random_model)
from tests.helpers import TINY_A, TINY_B, make_model_folder


def _model(cfg):
    _, typed = load_config(cfg)
    return typed, build_model(typed, torch.float32, "cpu")


def test_random_folder_roundtrip_and_names(tmp_path):
    folder = make_model_folder(tmp_path, TINY_B, seed=3)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(folder, "config.json")))["num_key_value_heads"] == 1
    typed, model = _model(TINY_B)
    w = load_weights(folder, model.param_specs(), torch.bfloat16, "cpu")
    assert w["model.layers.2.self_attn.q_proj.weight"].shape == (192, 192)
    assert w["model.layers.0.self_attn.k_proj.weight"].shape == (32, 192)
    assert w["model.layers.1.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert w["model.layers.1.self_attn.v_proj.bias"].dtype == torch.float32   # vectors: float32, exact
    assert w["lm_head.weight"].shape == (1000, 192)
    # the independent safetensors reader sees the same bytes
    from safetensors.torch import load_file
    ref = load_file(os.path.join(folder, "model.safetensors"))
    assert set(ref) == {p.name for p in model.param_specs() if not p.optional}
    for k in ref:
        assert torch.equal(ref[k].float(), w[k].float())
    # float32 run: exact upcast
    w32 = load_weights(folder, model.param_specs(), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["model.embed_tokens.weight"], ref["model.embed_tokens.weight"].float())


def test_random_mode_is_seeded(tmp_path):
    from safetensors.torch import load_file
    a = load_file(os.path.join(make_model_folder(tmp_path / "a", TINY_A, 5), "model.safetensors"))
    b = load_file(os.path.join(make_model_folder(tmp_path / "b", TINY_A, 5), "model.safetensors"))
    c = load_file(os.path.join(make_model_folder(tmp_path / "c", TINY_A, 6), "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert "lm_head.weight" not in a                     # tied: no separate head is written
    g = a["model.layers.0.input_layernorm.weight"].float()
    assert 0.5 < g.mean() < 1.5 and g.std() > 0.01       # gains are not the identity
    assert a["model.layers.0.self_attn.q_proj.bias"].float().abs().max() > 0


def test_stored_32bit_stays_32bit_and_ints_become_int32(tmp_path):
    specs = [ParamSpec("m.weight", (4, 6)), ParamSpec("n.weight", (4, 6)), ParamSpec("t.table", (5,), kind="int")]
    save_file({"m.weight": torch.randn(4, 6), "n.weight": torch.randn(4, 6).to(torch.bfloat16),
               "t.table": torch.arange(5, dtype=torch.int64)}, str(tmp_path / "model.safetensors"))
    w = load_weights(str(tmp_path), specs, torch.bfloat16, "cpu")
    assert w["m.weight"].dtype == torch.float32 and w["n.weight"].dtype == torch.bfloat16
    assert w["t.table"].dtype == torch.int32 and w["t.table"].tolist() == [0, 1, 2, 3, 4]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    folder = make_model_folder(tmp_path, TINY_A, seed=1)
    f = os.path.join(folder, "model.safetensors")
    w = load_file(f)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.int32)
    st_save(w, f)
    _, model = _model(TINY_A)
    with pytest.raises(WeightsError) as e:
        load_weights(folder, model.param_specs(), torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    assert err.wrong_dtype[0][0] == "model.layers.0.self_attn.q_proj.bias"
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "is [16, 64], expected [32, 64]"):
        assert needle in text


def test_tied_model_accepts_or_omits_lm_head(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    folder = make_model_folder(tmp_path, TINY_A, seed=1)
    _, model = _model(TINY_A)
    load_weights(folder, model.param_specs(), torch.float32, "cpu")
    f = os.path.join(folder, "model.safetensors")
    w = load_file(f)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    st_save(w, f)
    out = load_weights(folder, model.param_specs(), torch.float32, "cpu")
    model.load(out)
    assert model.lm_head is model.embed


def test_untied_model_needs_lm_head(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    folder = make_model_folder(tmp_path, TINY_B, seed=1)
    f = os.path.join(folder, "model.safetensors")
    w = load_file(f)
    del w["lm_head.weight"]
    st_save(w, f)
    _, model = _model(TINY_B)
    with pytest.raises(WeightsError) as e:
        load_weights(folder, model.param_specs(), torch.float32, "cpu")
    assert e.value.missing == ["lm_head.weight"]


def test_broken_files(tmp_path):
    _, model = _model(TINY_A)
    with pytest.raises(WeightsError):
        load_weights(str(tmp_path), model.param_specs(), torch.float32, "cpu")   # no file
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00\x00")
    with pytest.raises(WeightsError):
        load_weights(str(tmp_path), model.param_specs(), torch.float32, "cpu")
    (tmp_path / "model.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightsError):
        load_weights(str(tmp_path), model.param_specs(), torch.float32, "cpu")


def test_fused_layouts_after_load(tmp_path):
    folder = make_model_folder(tmp_path, TINY_B, seed=2)
    _, model = _model(TINY_B)
    w = load_weights(folder, model.param_specs(), torch.float32, "cpu")
    model.load(w)
    attn = model.blocks[0].mixer
    assert attn.w_qkv.shape == (6 * 32 + 2 * 32, 192) and attn.b_qkv.shape == (256,)
    assert torch.equal(attn.w_qkv[192:224], w["model.layers.0.self_attn.k_proj.weight"])
    ffn = model.blocks[2].ffn
    assert ffn.w_gate_up.shape == (1024, 192)
    assert torch.equal(ffn.w_gate_up[512:], w["model.layers.2.mlp.up_proj.weight"])
