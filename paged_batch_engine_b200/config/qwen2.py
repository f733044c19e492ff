"""Typed configuration of the Qwen2 / Qwen2.5 dense decoder, read from config.json.

The reference engine reads seven integers from a binary header and hard-codes the
rest (infMain/include/model/config.h:5-42; theta in
infMain/source/op/kernels/cuda/rope_kernel.cu:78-80; eps in
infMain/source/op/kernels/cuda/rmsnorm_kernel.cu:127).  Here every one of them is a
field read from the architecture's own ``config.json`` keys, the ones the
reference's exporter reads (tools/export_qwen2.py:626-634) plus those it drops.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep

_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
             "intermediate_size", "vocab_size")


@dataclass
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    head_dim: Optional[int] = None           # default hidden_size / num_attention_heads
    rms_norm_eps: float = 1e-6                # the reference's fixed value when the key is absent
    rope_theta: float = 1000000.0             # the reference's fixed value when the key is absent
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    hidden_act: str = "silu"
    rope_scaling: Optional[dict] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Any = None                  # int, list of ints or None
    torch_dtype: str = "bfloat16"
    architectures: List[str] = field(default_factory=lambda: ["Qwen2ForCausalLM"])
    model_type: str = "qwen2"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {', '.join(missing)}")
        known = {f for f in cls.__dataclass_fields__}
        kwargs = {k: v for k, v in d.items() if k in known}
        if "dtype" in d and "torch_dtype" not in d:
            kwargs["torch_dtype"] = d["dtype"]
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen2Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["head_dim"] = self.resolved_head_dim
        return d

    # ------------------------------------------------------------------ derived
    @property
    def resolved_head_dim(self) -> int:
        if self.head_dim is not None:
            return int(self.head_dim)
        return self.hidden_size // self.num_attention_heads

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        e = self.eos_token_id
        if e is None:
            return ()
        if isinstance(e, (list, tuple)):
            return tuple(int(x) for x in e)
        return (int(e),)

    def layer_window(self, layer: int) -> Optional[int]:
        """Layers with index >= max_window_layers attend to the last ``sliding_window``
        keys when ``use_sliding_window`` is set; all others to every key.  The
        reference engine never windows (it visits keys 0..p for every query,
        infMain/source/op/kernels/cuda/paged_mha_kernel.cu:444-480)."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return int(self.sliding_window) if layer >= first else None

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        def positive(name):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        for name in _REQUIRED + ("max_position_embeddings",):
            positive(name)
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim is None and self.hidden_size % self.num_attention_heads != 0:
            raise ConfigError(
                f"hidden_size ({self.hidden_size}) is not a multiple of num_attention_heads "
                f"({self.num_attention_heads}) and head_dim is not given")
        hd = self.resolved_head_dim
        if hd <= 0 or hd % 2 != 0:
            raise ConfigError(f"head_dim must be positive and even for rotate-half RoPE, got {hd}")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.rope_scaling not in (None, {}):
            kind = (self.rope_scaling or {}).get("rope_type", (self.rope_scaling or {}).get("type"))
            if kind not in (None, "default"):
                raise ConfigError(f"rope_scaling {self.rope_scaling!r} is not supported")
        if self.use_sliding_window:
            if self.sliding_window is None or int(self.sliding_window) <= 0:
                raise ConfigError("use_sliding_window is set but sliding_window is not a positive integer")
            if self.max_window_layers is not None and self.max_window_layers < 0:
                raise ConfigError("max_window_layers must be >= 0")

    # ------------------------------------------------------------------ the model as data
    def model_spec(self) -> ModelSpec:
        hd = self.resolved_head_dim
        blocks = []
        for i in range(self.num_hidden_layers):
            rope = PartSpec("rope", dict(theta=float(self.rope_theta), head_dim=hd, rotary_dim=hd,
                                         pairing="half"))
            mixer = PartSpec("attention", dict(
                hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads, head_dim=hd, qkv_bias=True, o_bias=False,
                scale=hd ** -0.5, window=self.layer_window(i), position=rope))
            ffn = PartSpec("swiglu", dict(hidden_size=self.hidden_size,
                                          intermediate_size=self.intermediate_size))
            norm = PartSpec("rmsnorm", dict(size=self.hidden_size, eps=float(self.rms_norm_eps)))
            blocks.append(BlockSpec(
                kind="prenorm", mixer=mixer, feed_forward=ffn, norm_mixer=norm,
                norm_feed_forward=norm, prefix=f"model.layers.{i}.",
                names=dict(mixer="self_attn.", feed_forward="mlp.", norm_mixer="input_layernorm.",
                           norm_feed_forward="post_attention_layernorm.")))
        run = tuple(RunStep(block=i, cache_layer=i) for i in range(self.num_hidden_layers))
        return ModelSpec(
            architecture="Qwen2ForCausalLM", hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, blocks=tuple(blocks), run_order=run,
            final_norm=PartSpec("rmsnorm", dict(size=self.hidden_size, eps=float(self.rms_norm_eps))),
            embedding_name="model.embed_tokens.weight", final_norm_name="model.norm.",
            lm_head_name=None if self.tie_word_embeddings else "lm_head.weight",
            max_position=self.max_position_embeddings, eos_token_ids=self.eos_token_ids)
