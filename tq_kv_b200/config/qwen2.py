"""Typed configuration of the Qwen2 / Qwen2.5 dense decoder, read from the
keys of that architecture's config.json, and the builder that turns it into a
`ModelSpec` of parts.

Reference: src/models/turbo_generic.rs:2013-2030 reads the same keys untyped
and with silent defaults (heads 32, layers 32, hidden 4096, ...); here a
missing size is an error.  The formulas the parts follow are cited in the
parts themselves.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Optional

from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Qwen2ForCausalLM"
MODEL_TYPE = "qwen2"

_MISSING = object()


def _get(d: dict, key: str, typ, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key '{key}'")
        return default
    v = d[key]
    if typ is float and isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    if typ is int and isinstance(v, int) and not isinstance(v, bool):
        return int(v)
    if typ is bool and isinstance(v, bool):
        return v
    if typ is str and isinstance(v, str):
        return v
    raise ConfigError(f"config.json: key '{key}' should be {typ.__name__}, found {v!r}")


@dataclass(frozen=True)
class Qwen2Config:
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
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    hidden_act: str
    eos_token_ids: tuple[int, ...]
    bos_token_id: Optional[int]
    torch_dtype: str

    # ---- reading -------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen2Config":
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        layers = _get(d, "num_hidden_layers", int)
        # src/models/turbo_generic.rs:2014 — KV heads default to the head count,
        # :2020-2022 — head_dim defaults to hidden / heads.
        kv_heads = _get(d, "num_key_value_heads", int, heads)
        if heads <= 0 or hidden <= 0 or layers <= 0:
            raise ConfigError("config.json: sizes must be positive")
        head_dim = _get(d, "head_dim", int, None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and no head_dim is given")
            head_dim = hidden // heads
        use_window = _get(d, "use_sliding_window", bool, False)
        window = _get(d, "sliding_window", int, None)
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: key 'eos_token_id' should be int or list of int, found {eos!r}")
        cfg = cls(
            vocab_size=_get(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_get(d, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_get(d, "max_position_embeddings", int),
            rms_norm_eps=_get(d, "rms_norm_eps", float),
            rope_theta=_get(d, "rope_theta", float),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=_get(d, "max_window_layers", int, layers),
            hidden_act=_get(d, "hidden_act", str, "silu"),
            eos_token_ids=eos_ids,
            bos_token_id=_get(d, "bos_token_id", int, None),
            torch_dtype=_get(d, "torch_dtype", str, "bfloat16"),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "Qwen2Config":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ConfigError(f"config.json: head_dim {self.head_dim} is not supported: the attention kernels take "
                              "head sizes that are multiples of 16 from 16 to 256")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("config.json: use_sliding_window is true but sliding_window is missing or <= 0")
        for name in ("vocab_size", "intermediate_size", "max_position_embeddings", "num_key_value_heads"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: '{name}' must be positive")
        if not (self.rms_norm_eps > 0.0 and self.rope_theta > 0.0):
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")

    # ---- writing (the random-weights mode writes a model folder) --------
    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architectures": [ARCHITECTURE],
            "model_type": MODEL_TYPE,
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
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # ---- the window rule -------------------------------------------------
    def layer_window(self, layer: int) -> Optional[int]:
        """Window of layer `layer`, or None for plain causal attention.  The
        reference has no sliding window in code; the rule here is: a layer is
        windowed iff use_sliding_window and layer >= max_window_layers, and a
        windowed query at position p sees keys max(0, p - window + 1) .. p."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None


def read_config_json(path: str) -> dict[str, Any]:
    """Reads config.json given the file or its folder.  Error texts follow
    src/models/turbo_generic.rs:2008-2011."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            text = f.read()
    except OSError as e:
        raise ConfigError(f"Cannot read config.json: {e}") from e
    try:
        d = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"Invalid config.json: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError("Invalid config.json: top level is not an object")
    return d


def build_qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    """Qwen2 as parts: token embedding; per layer a pre-norm residual block of
    {RMSNorm, grouped-query attention with q/k/v bias and rotate-half rotary
    positions, RMSNorm, SwiGLU}; final RMSNorm; LM head tied to the embedding
    or with a matrix of its own."""
    norm = {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps}
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qkv_bias": True,            # src/models/turbo_generic.rs:805-813
            "out_bias": False,           # :1633-1634, no o_proj bias is ever looked up
            "window": cfg.layer_window(i),
            "position": PartSpec("rotary_halved", {
                "head_dim": cfg.head_dim,
                "rotary_dim": cfg.head_dim,  # :2030, the full head is rotated
                "theta": cfg.rope_theta,
            }),
            "names": {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"},
        }, p + "self_attn.")
        ffn = PartSpec("swiglu", {
            "hidden_size": cfg.hidden_size,
            "intermediate_size": cfg.intermediate_size,
            "names": {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"},
        }, p + "mlp.")
        layers.append(LayerSpec(
            block="prenorm_residual",
            mixer=mixer,
            feed_forward=ffn,
            mixer_norm=PartSpec("rms_norm", dict(norm), p + "input_layernorm."),
            feed_forward_norm=PartSpec("rms_norm", dict(norm), p + "post_attention_layernorm."),
        ))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": cfg.hidden_size},
                           "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", dict(norm), "model.norm."),
        head=PartSpec("lm_head", {
            "vocab_size": cfg.vocab_size, "width": cfg.hidden_size,
            "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
        }, "lm_head."),
        stop_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec
