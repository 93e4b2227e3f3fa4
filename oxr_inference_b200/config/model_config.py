"""Typed configuration read from a model folder's ``config.json``.

Every size and constant of the network comes from here; nothing in the model code carries a number that
``config.json`` gives. The reference reads the same nine language-model keys, all required, from the
``llm_config`` sub-dict of its wrapper config (oxr_runtime/config.py:90-100) and the end-of-sequence ids from
``generation_config.json`` first, then ``config.json`` (oxr_runtime/config.py:68-74). A plain Qwen3 folder
keeps those keys at the top level; both placements are accepted.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine does not implement."""


_REQUIRED = (
    "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
    "rms_norm_eps", "rope_theta", "vocab_size",
)

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config:
    """The Qwen3 dense decoder's own config.json keys (field names are the json keys)."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    vocab_size: int
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str
    attention_bias: bool
    sliding_window: int | None
    layer_types: tuple[str, ...]
    eos_token_ids: tuple[int, ...]
    torch_dtype: str
    architecture: str = "Qwen3ForCausalLM"

    # ---- derived sizes -------------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def window_of(self, layer: int) -> int:
        """Keys a query of this layer may see, itself included; 0 means all of them."""
        if self.layer_types[layer] == SLIDING_ATTENTION:
            assert self.sliding_window is not None
            return self.sliding_window
        return 0

    # ---- reading -------------------------------------------------------------------------------------
    @staticmethod
    def from_dict(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "Qwen3Config":
        llm = raw.get("llm_config", raw)  # the reference nests the keys (oxr_runtime/config.py:66)
        missing = [k for k in _REQUIRED if k not in llm]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")

        def positive_int(key: str, value: Any) -> int:
            if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
                raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
            return value

        hidden = positive_int("hidden_size", llm["hidden_size"])
        heads = positive_int("num_attention_heads", llm["num_attention_heads"])
        kv_heads = positive_int("num_key_value_heads", llm["num_key_value_heads"])
        layers = positive_int("num_hidden_layers", llm["num_hidden_layers"])
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        head_dim = llm.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"no head_dim given and hidden_size {hidden} is not a multiple of {heads} heads")
            head_dim = hidden // heads
        head_dim = positive_int("head_dim", head_dim)
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} is odd; rotary position encoding needs pairs")

        if llm.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not implemented (the reference has no biases, "
                              "oxr_runtime/language.py:223-231)")
        act = llm.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not implemented; the feed-forward is SiLU-gated")
        scaling = llm.get("rope_scaling")
        if scaling not in (None, {}) and scaling.get("rope_type", scaling.get("type")) not in (None, "default"):
            raise ConfigError(f"rope_scaling {scaling!r} is not implemented")

        window = llm.get("sliding_window")
        use_window = bool(llm.get("use_sliding_window", False))
        types = llm.get("layer_types")
        if types is None:
            first_windowed = llm.get("max_window_layers", layers) if (use_window and window) else layers
            types = [SLIDING_ATTENTION if i >= first_windowed else FULL_ATTENTION for i in range(layers)]
        types = tuple(types)
        if len(types) != layers:
            raise ConfigError(f"layer_types has {len(types)} entries for {layers} layers")
        unknown = sorted(set(types) - {FULL_ATTENTION, SLIDING_ATTENTION})
        if unknown:
            raise ConfigError(f"layer_types holds unknown kinds {unknown}")
        if SLIDING_ATTENTION in types:
            window = positive_int("sliding_window", window)
        else:
            window = None

        eos: list[int] = []
        if generation is not None:
            value = generation.get("eos_token_id", [])
            eos = list(value) if isinstance(value, list) else [value]
        if not eos:
            value = raw.get("eos_token_id", llm.get("eos_token_id", []))
            if value is None:
                value = []
            eos = list(value) if isinstance(value, list) else [value]

        archs = raw.get("architectures") or ["Qwen3ForCausalLM"]
        return Qwen3Config(
            hidden_size=hidden,
            intermediate_size=positive_int("intermediate_size", llm["intermediate_size"]),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(llm["rms_norm_eps"]),
            rope_theta=float(llm["rope_theta"]),
            vocab_size=positive_int("vocab_size", llm["vocab_size"]),
            # The reference sizes its rotary table from an engine setting of 40960 (oxr_runtime/engine.py:115);
            # a Qwen3 config.json carries the same number under this key.
            max_position_embeddings=positive_int("max_position_embeddings", llm.get("max_position_embeddings", 40960)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", llm.get("tie_word_embeddings", False))),
            hidden_act=act,
            attention_bias=False,
            sliding_window=window,
            layer_types=types,
            eos_token_ids=tuple(int(t) for t in eos),
            torch_dtype=str(llm.get("torch_dtype", llm.get("dtype", "bfloat16"))),
            architecture=str(archs[0]),
        )

    def to_dict(self) -> dict[str, Any]:
        """A config.json that reads back to this object."""
        out: dict[str, Any] = {"architectures": [self.architecture], "model_type": "qwen3"}
        skip = {"architecture", "eos_token_ids", "layer_types", "sliding_window"}
        for f in fields(self):
            if f.name not in skip:
                out[f.name] = getattr(self, f.name)
        if self.sliding_window is not None:
            out["sliding_window"] = self.sliding_window
            out["use_sliding_window"] = True
            out["layer_types"] = list(self.layer_types)
        else:
            out["sliding_window"] = None
            out["use_sliding_window"] = False
        if self.eos_token_ids:
            out["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return out


def read_config_json(model_dir: str | Path) -> tuple[dict[str, Any], dict[str, Any] | None]:
    root = Path(model_dir)
    path = root / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    raw = json.loads(path.read_text())
    generation = root / "generation_config.json"
    return raw, (json.loads(generation.read_text()) if generation.is_file() else None)


def load_model_config(model_dir: str | Path):
    """Read ``config.json`` and return ``(architecture, typed config)``; the architecture is looked up in the
    registry by the first entry of ``architectures``."""
    from oxr_inference_b200.config.registry import resolve_architecture

    raw, generation = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    return arch, arch.config_from_dict(raw, generation)
