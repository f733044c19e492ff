"""Shared test data: tiny configurations and model-folder helpers."""
import json
import os

import torch

# Tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=64,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=160,
              vocab_size=320, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=4096, use_sliding_window=False, hidden_act="silu",
              eos_token_id=319)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=192,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, intermediate_size=512,
              vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=2048, use_sliding_window=False, hidden_act="silu",
              eos_token_id=[998, 999])
# head_dim given and unequal to hidden/heads, three kv heads, a window on layers 1.., sizes
# that are no power of two
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=88,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              intermediate_size=208, vocab_size=517, rope_theta=50000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=1024, use_sliding_window=True,
              sliding_window=24, max_window_layers=1, hidden_act="silu", eos_token_id=516)
# head size 64 (in bfloat16 its prompt portions run on the tcgen05 attention kernel), three
# query heads on one key/value head, a window on the second layer
TINY_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=96,
              num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1, head_dim=64,
              intermediate_size=144, vocab_size=411, rope_theta=20000.0, rms_norm_eps=2e-6,
              tie_word_embeddings=True, max_position_embeddings=2048, use_sliding_window=True,
              sliding_window=150, max_window_layers=1, hidden_act="silu", eos_token_id=410)
TINY = {"A": (TINY_A, 0, 16, 8.0), "B": (TINY_B, 1, 8, 4.0), "C": (TINY_C, 2, 8, 6.0), "D": (TINY_D, 3, 16, 5.0)}


def make_model_folder(path, cfg: dict, seed: int, sharpen: float = 1.0, dtype=torch.bfloat16) -> str:
    """A model folder with seeded random weights through the engine's random-weights mode;
    ``sharpen`` scales the query and key projections so that attention is far from uniform
    and a wrong, missing or extra key changes the logits visibly."""
    from paged_batch_engine_b200.config import load_config
    from paged_batch_engine_b200.engine.runner import build_model
    from paged_batch_engine_b200.weights import write_random_model
    _, typed = load_config(cfg)
    model = build_model(typed, torch.float32, "cpu")
    write_random_model(str(path), typed, model.param_specs(), seed, dtype)
    if sharpen != 1.0:
        from safetensors.torch import load_file, save_file
        f = os.path.join(str(path), "model.safetensors")
        w = load_file(f)
        for k in list(w):
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                w[k] = (w[k].float() * sharpen).to(w[k].dtype)
        save_file(w, f)
    return str(path)


def load_plain(folder: str):
    """config.json as a dict and the weights as float32 tensors, read without the engine."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


