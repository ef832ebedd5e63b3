"""Qwen3 dense: the typed configuration and its translation into parts.

Keys and checks follow the reference's parser (src/qwen/qwen_configs.cc:261-331):
the geometry keys, ``rms_norm_eps`` and ``rope_theta`` are required;
``model_type`` must be "qwen3", ``hidden_act`` "silu", ``attention_bias``
false, ``rope_scaling`` null.  Differences, all of them widenings:

* the offending key is named in the error;
* ``torch_dtype``/``dtype`` may also be "float32" (small 32-bit fixtures);
* ``bos_token_id``/``eos_token_id`` may be absent (random-weight models);
* ``head_dim`` may be absent and is then hidden_size / num_attention_heads;
* ``tie_word_embeddings`` may be absent and is then false;
* a sliding window is accepted (the reference refuses it,
  qwen_configs.cc:310-311): with ``use_sliding_window`` true, layers whose
  index is at least ``max_window_layers`` (or that ``layer_types`` marks
  "sliding_attention") see only the ``sliding_window`` most recent keys.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .base import ConfigError, KeyReader
from .spec import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                   PositionSpec, RunStep)

ARCHITECTURE = "Qwen3ForCausalLM"
MODEL_TYPE = "qwen3"


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    # one entry per layer: None (all keys) or the window length
    layer_windows: Tuple[Optional[int], ...] = field(default=())

    # ---- derived sizes (src/qwen/qwen_configs.cc:416-432) ----
    @property
    def query_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def queries_per_kv_head(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- reading ----
    @classmethod
    def from_dict(cls, obj: dict) -> "Qwen3Config":
        r = KeyReader(obj)
        for key in ("quantization", "quantization_config"):
            if r.has(key):
                raise ConfigError("unsupported_configuration",
                                  f"key '{key}': quantized checkpoints are not supported")
        r.require_value("model_type", (MODEL_TYPE,), code="unsupported_model_type")
        r.require_value("hidden_act", ("silu",))
        r.require_value("attention_bias", (False,), default=False)
        r.require_null_or_missing("rope_scaling")
        dtype_key = "torch_dtype" if r.has("torch_dtype") else "dtype"
        torch_dtype = r.require_value(dtype_key, ("bfloat16", "float32"), default="bfloat16")

        vocab = r.positive_int("vocab_size")
        hidden = r.positive_int("hidden_size")
        inter = r.positive_int("intermediate_size")
        layers = r.positive_int("num_hidden_layers")
        nq = r.positive_int("num_attention_heads")
        nkv = r.positive_int("num_key_value_heads")
        if r.has("head_dim"):
            head_dim = r.positive_int("head_dim")
        else:
            if hidden % nq != 0:
                raise ConfigError("invalid_geometry",
                                  "key 'head_dim' is absent and hidden_size is not a multiple of "
                                  "num_attention_heads")
            head_dim = hidden // nq
        max_pos = r.positive_int("max_position_embeddings")
        eps = r.positive_float("rms_norm_eps")
        if r.has("rope_theta"):
            theta = r.positive_float("rope_theta")
        elif r.has("rope_parameters"):
            rp = KeyReader(r.raw("rope_parameters"))
            rp.require_value("rope_type", ("default",), default="default")
            theta = rp.positive_float("rope_theta")
        else:
            raise ConfigError("missing_field", "key 'rope_theta' is required")
        bos = r.token_id("bos_token_id")
        eos = r.token_id("eos_token_id")
        tie = r.boolean("tie_word_embeddings", default=False)

        if nq % nkv != 0:
            raise ConfigError("invalid_geometry",
                              f"num_attention_heads {nq} is not a multiple of num_key_value_heads {nkv}")
        if head_dim % 2 != 0:
            raise ConfigError("invalid_geometry", f"head_dim {head_dim} must be even")
        for name, tok in (("bos_token_id", bos), ("eos_token_id", eos)):
            if tok is not None and tok >= vocab:
                raise ConfigError("invalid_geometry", f"key '{name}' {tok} is outside the vocabulary {vocab}")

        windows = cls._read_windows(r, layers)
        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                   num_hidden_layers=layers, num_attention_heads=nq, num_key_value_heads=nkv,
                   head_dim=head_dim, max_position_embeddings=max_pos, rms_norm_eps=eps,
                   rope_theta=theta, tie_word_embeddings=tie, bos_token_id=bos, eos_token_id=eos,
                   torch_dtype=torch_dtype, layer_windows=windows)

    @staticmethod
    def _read_windows(r: KeyReader, layers: int) -> Tuple[Optional[int], ...]:
        use = r.boolean("use_sliding_window", default=False)
        if not use:
            if r.has("layer_types"):
                types = r.raw("layer_types")
                if not isinstance(types, list) or any(t != "full_attention" for t in types):
                    raise ConfigError("unsupported_configuration",
                                      "key 'layer_types' names sliding layers but 'use_sliding_window' is false")
            return tuple([None] * layers)
        window = r.positive_int("sliding_window")
        if r.has("layer_types"):
            types = r.raw("layer_types")
            if not isinstance(types, list) or len(types) != layers:
                raise ConfigError("invalid_field", f"key 'layer_types' must list {layers} layer kinds")
            out = []
            for t in types:
                if t == "full_attention":
                    out.append(None)
                elif t == "sliding_attention":
                    out.append(window)
                else:
                    raise ConfigError("unsupported_configuration", f"key 'layer_types' holds {t!r}")
            return tuple(out)
        first = r.raw("max_window_layers", layers)
        if isinstance(first, bool) or not isinstance(first, int) or first < 0:
            raise ConfigError("invalid_field", "key 'max_window_layers' must be a non-negative integer")
        return tuple(None if i < first else window for i in range(layers))

    # ---- writing (random-weight model folders) ----
    def to_dict(self) -> dict:
        d = {
            "architectures": [ARCHITECTURE],
            "model_type": MODEL_TYPE,
            "attention_bias": False,
            "hidden_act": "silu",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        windows = [w for w in self.layer_windows if w is not None]
        if windows:
            if len(set(windows)) != 1:
                raise ConfigError("unsupported_configuration", "config.json holds one window length")
            d["use_sliding_window"] = True
            d["sliding_window"] = windows[0]
            d["layer_types"] = ["full_attention" if w is None else "sliding_attention"
                                for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
            d["sliding_window"] = None
        return d

    # ---- translation into parts ----
    def model_spec(self) -> ModelSpec:
        """Pre-norm decoder of ``num_hidden_layers`` equal blocks
        (src/qwen/qwen_layer.cc:103-149): input norm, q/k/v projection,
        per-head RMSNorm of q and k, split-half rotation, paged attention,
        output projection plus residual, post-attention norm, SwiGLU plus
        residual; final norm and vocabulary projection on the wanted rows."""
        windows = self.layer_windows or tuple([None] * self.num_hidden_layers)
        hidden_norm = NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, 0.0)
        head_norm = NormSpec("rmsnorm", self.head_dim, self.rms_norm_eps, 0.0)
        rope = PositionSpec(kind="rope", head_dim=self.head_dim, rotary_dim=self.head_dim,
                            theta=self.rope_theta)
        layers = []
        for i in range(self.num_hidden_layers):
            attn = AttentionSpec(
                kind="attention", hidden_size=self.hidden_size,
                num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim, scale=1.0 / math.sqrt(float(self.head_dim)),
                window=windows[i], qk_norm=head_norm, position=rope)
            mlp = GatedMLPSpec(kind="gated_mlp", hidden_size=self.hidden_size,
                               intermediate_size=self.intermediate_size, activation="silu")
            layers.append(LayerSpec(
                arrangement="prenorm", mixer=attn, feed_forward=mlp,
                mixer_norm=hidden_norm, feed_forward_norm=hidden_norm,
                weight_prefix=f"model.layers.{i}.",
                weight_names=(
                    ("mixer_norm", "input_layernorm.weight"),
                    ("feed_forward_norm", "post_attention_layernorm.weight"),
                    ("q_proj", "self_attn.q_proj.weight"),
                    ("k_proj", "self_attn.k_proj.weight"),
                    ("v_proj", "self_attn.v_proj.weight"),
                    ("o_proj", "self_attn.o_proj.weight"),
                    ("q_norm", "self_attn.q_norm.weight"),
                    ("k_norm", "self_attn.k_norm.weight"),
                    ("gate_proj", "mlp.gate_proj.weight"),
                    ("up_proj", "mlp.up_proj.weight"),
                    ("down_proj", "mlp.down_proj.weight"),
                )))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings, layers=tuple(layers),
            run_order=tuple(RunStep(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=hidden_norm, embedding_name="model.embed_tokens.weight",
            final_norm_name="model.norm.weight", output_name="lm_head.weight",
            tie_output_to_embedding=self.tie_word_embeddings,
            eos_token_id=self.eos_token_id, bos_token_id=self.bos_token_id)
