"""Grouped-query attention over the paged cache, with optional per-head q/k RMSNorm, rotary encoding and window."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import (MIXERS, DeferredLinear, LayerCache, Mixer, PagedKVNeed, ParamInfo, PositionEncoding, Runtime,
                                           StepContext)
from oxr_inference_b200.parts.linear import StackedLinear


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    """``qkv = h W_qkv^T`` -> per-head RMSNorm of q and k -> rotary -> K, V into the cache -> causal softmax
    attention of the new tokens over the cached keys -> ``W_o`` (oxr_runtime/language.py:247-264,271-299).

    All sizes and constants are arguments: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``
    (the reference fixes head_dim**-0.5, language.py:232), ``qk_norm`` with its ``eps``, ``window`` (0 = none).
    """

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int,
                 num_kv_heads: int, head_dim: int, scale: float, qk_norm: bool = True, eps: float = 1e-6,
                 window: int = 0):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} KV heads")
        ops.build.check_head_dim(head_dim)
        self.runtime = runtime
        self.hidden, self.H, self.KV, self.D = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.qk_norm, self.eps, self.window = float(scale), bool(qk_norm), float(eps), int(window)
        self.position = position
        self.qkv = StackedLinear(runtime, self.hidden, {"q_proj.weight": self.H * self.D, "k_proj.weight": self.KV * self.D,
                                                        "v_proj.weight": self.KV * self.D})
        self.o_proj = StackedLinear(runtime, self.H * self.D, {"o_proj.weight": self.hidden})
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        out = {**self.qkv.parameters(), **self.o_proj.parameters()}
        if self.qk_norm:
            out["q_norm.weight"] = ParamInfo((self.D,), init="around_one", role="vector")
            out["k_norm.weight"] = ParamInfo((self.D,), init="around_one", role="vector")
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.qkv.outs:
            self.qkv.assign(name, tensor)
        elif name in self.o_proj.outs:
            self.o_proj.assign(name, tensor)
        elif name == "q_norm.weight" and self.qk_norm:
            self.q_norm = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        elif name == "k_norm.weight" and self.qk_norm:
            self.k_norm = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.KV, self.D, self.window)

    def tile_specs(self) -> list[tuple[int, int, int]]:
        return ops.attention_tile_specs(self.H, self.KV, self.D, self.runtime.dtype, self.runtime.page_size)

    accepts_lazy_input = True   # h goes into the q|k|v projection and nowhere else

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.o_proj(self._attend(h, ctx, cache))

    def forward_deferred(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> DeferredLinear:
        return DeferredLinear(self._attend(h, ctx, cache), self.o_proj)

    def _attend(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """Everything up to the output projection: ``[tokens, H * D]``."""
        group = cache.group
        k_pool, v_pool = group.k_pool[cache.layer_in_group], group.v_pool[cache.layer_in_group]
        qkv = self.qkv(h)
        if qkv.dtype != k_pool.dtype:  # weights kept in 32-bit under 16-bit activations
            qkv = ops.cast(qkv, k_pool.dtype)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        if ctx.single_tokens and ops.attention_takes_projections(self.D, qkv.dtype, group.page_size, group.kv_maps, requests=ctx.n_requests,
                                                                 num_heads=self.H, num_kv_heads=self.KV, kv_len_bound=ctx.kv_len_bound,
                                                                 uneven=ctx.uneven):
            # a decode step: the attention kernel normalises, rotates and stores the one new token of each request itself
            o = ops.decode_attention_from_projections(
                qkv, self.q_norm, self.k_norm, cos, sin, k_pool, v_pool, store=cache.store, num_heads=self.H, num_kv_heads=self.KV,
                head_dim=self.D, eps=self.eps, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens, block_table=group.block_table,
                page_size=group.page_size, scale=self.scale, window=self.window, kv_len_bound=ctx.kv_len_bound, status=ctx.status,
                kv_maps=group.kv_maps, layer_in_pool=cache.layer_in_group, uneven=ctx.uneven)
            return o.view(ctx.n_tokens, self.H * self.D)
        q = ops.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, cos, sin, ctx.positions,
                                   group.slots if cache.store else ctx.no_store_slots, k_pool, v_pool,
                                   self.H, self.KV, self.D, self.eps, ctx.status)
        o = ops.paged_attention(q, k_pool, v_pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens,
                                block_table=group.block_table, page_size=group.page_size, scale=self.scale,
                                window=self.window, kv_len_bound=ctx.kv_len_bound, status=ctx.status,
                                kv_maps=group.kv_maps, layer_in_pool=cache.layer_in_group, uneven=ctx.uneven)
        return o.view(ctx.n_tokens, self.H * self.D)
