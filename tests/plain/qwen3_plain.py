"""Plain, slow implementation of the Qwen3 dense decoder: whole sequences, dense mask, no cache, one function
per part. It is the oracle of the tests and shares no code with the engine (it does not import it).

Written from the reference's formulas; each function cites where (paths inside NickWilde18/oxr-inference).
``tests/golden/make_reference_golden.py`` compared it once, on the CPU, with the reference's own
``LanguageModel`` on a tiny random model; the committed outputs are under ``tests/golden/``. The sliding window
(`layer_types` / `sliding_window` of a Qwen3 config.json) has no counterpart in the reference, whose layers all
see every earlier key; for it this file rests on the rule "a query at position p sees keys p - window < j <= p".
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F
from safetensors.torch import load_file


def read_model(folder: str | Path, dtype: torch.dtype = torch.float32):
    """config.json as a dict and all tensors by name, widened to ``dtype``."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {k: v.to(dtype) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, weights


def head_dim_of(cfg: dict) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def window_of(cfg: dict, layer: int) -> int:
    """Keys a query of this layer sees, itself included; 0 = all."""
    types = cfg.get("layer_types")
    if types is None:
        if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
            return cfg["sliding_window"] if layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]) else 0
        return 0
    return cfg["sliding_window"] if types[layer] == "sliding_attention" else 0


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """oxr_runtime/language.py:69-72: ``x * rsqrt(mean(x^2, -1) + eps)`` times the weight."""
    return weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))


def rope_tables(head_dim: int, theta: float, n: int, dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """oxr_runtime/language.py:160-165: fp32 inv_freq = 1 / theta^(2i/D), freqs = position (x) inv_freq, cos/sin.
    The table is made in fp32 as the reference makes it, then widened if the caller computes in fp64."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    freqs = torch.outer(torch.arange(n, dtype=torch.float), inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def rotate_half_split(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """oxr_runtime/language.py:84-91, oxr_runtime/kernels.py:61-63: x is [n, heads, D]; with x1, x2 the two halves of
    the last axis, out = (x1 c - x2 s, x1 s + x2 c)."""
    half = cos.shape[-1]
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0) -> torch.Tensor:
    """tests/test_language_fused.py:19-28,110-115 (the reference's own plain attention): q [n, H, D], k and v
    [n, KV, D]; q head j uses KV head j // (H / KV); scores = q k^T * scale; key j is masked for query i when j > i
    (and, with a window, when j <= i - window); softmax over keys; weighted sum of v."""
    n, H, _ = q.shape
    rep = H // k.shape[1]
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("nhd,mhd->hnm", q, k) * scale
    i = torch.arange(n, device=q.device)[:, None]
    j = torch.arange(n, device=q.device)[None, :]
    hidden = j > i
    if window > 0:
        hidden = hidden | (j <= i - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    return torch.einsum("hnm,mhd->nhd", scores.softmax(-1), v)


def swiglu(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """oxr_runtime/language.py:102-104,266-269: down( silu(h Wg^T) * (h Wu^T) ), no biases."""
    return (F.silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def attention_block(h: torch.Tensor, w: dict, prefix: str, cfg: dict, cos, sin, window: int) -> torch.Tensor:
    """oxr_runtime/language.py:247-264,271-283: projections (no bias), per-head RMSNorm of q and k over head_dim with
    one weight for all heads (oxr_runtime/kernels.py:48-60), rotary on q and k, attention with scale
    head_dim^-0.5 (language.py:232), output projection."""
    n = h.shape[0]
    H, KV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    eps = cfg["rms_norm_eps"]
    q = (h @ w[prefix + "q_proj.weight"].T).view(n, H, D)
    k = (h @ w[prefix + "k_proj.weight"].T).view(n, KV, D)
    v = (h @ w[prefix + "v_proj.weight"].T).view(n, KV, D)
    q = rotate_half_split(rms_norm(q, w[prefix + "q_norm.weight"], eps), cos, sin)
    k = rotate_half_split(rms_norm(k, w[prefix + "k_norm.weight"], eps), cos, sin)
    a = causal_attention(q, k, v, D ** -0.5, window)
    return a.reshape(n, H * D) @ w[prefix + "o_proj.weight"].T


def decoder_layer(x: torch.Tensor, w: dict, layer: int, cfg: dict, cos, sin) -> torch.Tensor:
    """tests/test_language_fused.py:104-119 (same sums as oxr_runtime/language.py:184-187,266-269):
    x += attention(norm(x)); x += mlp(norm(x))."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p + "self_attn.", cfg, cos, sin, window_of(cfg, layer))
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    return x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def hidden_states(cfg: dict, w: dict, ids: list[int]) -> torch.Tensor:
    """Final-norm hidden state of every position of one whole sequence (oxr_runtime/language.py:177-187)."""
    dtype = w["model.embed_tokens.weight"].dtype
    x = w["model.embed_tokens.weight"][torch.tensor(ids, dtype=torch.long)]
    cos, sin = (t.to(x.device) for t in rope_tables(head_dim_of(cfg), cfg["rope_theta"], len(ids), dtype))
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, cos, sin)
    return rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])


def logits(cfg: dict, w: dict, ids: list[int]) -> torch.Tensor:
    """[len(ids), vocab]: the output head on every position (oxr_runtime/language.py:213-214); a tied model
    multiplies by the embedding table."""
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return hidden_states(cfg, w, ids) @ head.T


def greedy(cfg: dict, w: dict, prompt: list[int], steps: int) -> list[int]:
    """Greedy decoding by recomputing the whole sequence for each new token (first maximum, as argmax does)."""
    ids, out = list(prompt), []
    for _ in range(steps):
        nxt = int(logits(cfg, w, ids)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
