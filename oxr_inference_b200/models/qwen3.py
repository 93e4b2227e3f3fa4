"""Qwen3 dense decoder: from its typed config to a description made of registered parts.

The structure is the one ``oxr_runtime/language.py`` runs: pre-norm blocks of grouped-query attention (per-head
q/k RMSNorm, half-split rotary, scale head_dim**-0.5, no biases) and a SiLU-gated feed-forward, a final RMSNorm
and an output head (language.py:149-317). Tensor names are the checkpoint's, as the reference maps them
(oxr_runtime/weight_names.py:25-32), with or without its ``llm.`` prefix.
"""

from __future__ import annotations

from oxr_inference_b200.config.model_config import Qwen3Config
from oxr_inference_b200.config.registry import Architecture, register_architecture
from oxr_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def qwen3_model_spec(c: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rope_neox", {"dim": c.head_dim, "theta": c.rope_theta})
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer=PartSpec("gqa_attention", {
                "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads, "num_kv_heads": c.num_key_value_heads,
                "head_dim": c.head_dim, "scale": c.head_dim ** -0.5, "qk_norm": True, "eps": c.rms_norm_eps,
                "window": c.window_of(i),
            }, prefix=p + "self_attn."),
            mixer_norm=PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps}, prefix=p + "input_layernorm."),
            feed_forward=PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size},
                                  prefix=p + "mlp."),
            feed_forward_norm=PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps},
                                       prefix=p + "post_attention_layernorm."),
            arrangement="pre_norm",
            position=rope,
        ))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size},
                           prefix="model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(c.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps}, prefix="model.norm."),
        head=PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
                                      "tied": c.tie_word_embeddings}, prefix="lm_head."),
        max_positions=c.max_position_embeddings,
        eos_token_ids=c.eos_token_ids,
        # a tied checkpoint may still carry a copy of the head
        ignored_tensors=(r"lm_head\.weight",) if c.tie_word_embeddings else (),
        name_prefixes=("", "llm."),
    )


QWEN3 = register_architecture(Architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_model_spec))
