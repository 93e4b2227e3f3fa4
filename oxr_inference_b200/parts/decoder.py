"""The decoder: embedding, a schedule of blocks, final norm, output head. Built from a ModelSpec alone."""

from __future__ import annotations

from typing import Any

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.cache.plan import CachePlan, make_cache_plan
from oxr_inference_b200.parts.base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                                           Embedding, Head, ParamInfo, Part, Runtime, StepContext)
from oxr_inference_b200.parts.spec import ModelSpec, PartSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """``x = table[ids]`` (oxr_runtime/language.py:155, oxr_runtime/decode_graph.py:75)."""

    def __init__(self, runtime: Runtime, *, vocab_size: int, hidden_size: int):
        self.runtime, self.vocab, self.hidden = runtime, int(vocab_size), int(hidden_size)
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {"weight": ParamInfo((self.vocab, self.hidden))}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight":
            raise KeyError(name)
        dtype = self.runtime.store_dtype(self.parameters()["weight"], tensor.dtype)
        self.weight = tensor.to(device=self.runtime.device, dtype=dtype).contiguous()

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids, self.weight, self.runtime.dtype, self.runtime.status)


@HEADS.register("linear_head")
class OutputHead(Head):
    """``logits = h W^T`` in fp32 (oxr_runtime/language.py:158,213-214). ``tied``: W is the embedding table, which
    the reference does not offer (its head is always a tensor of its own)."""

    def __init__(self, runtime: Runtime, embedding: Embedding, *, vocab_size: int, hidden_size: int, tied: bool):
        self.runtime, self.embedding = runtime, embedding
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {} if self.tied else {"weight": ParamInfo((self.vocab, self.hidden))}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight" or self.tied:
            raise KeyError(name)
        dtype = self.runtime.store_dtype(self.parameters()["weight"], tensor.dtype)
        self.weight = tensor.to(device=self.runtime.device, dtype=dtype).contiguous()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        w = self.embedding.weight if self.tied else self.weight
        return ops.linear(h, w, torch.float32)


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self._named: dict[str, tuple[Part, str, ParamInfo]] = {}
        self._positions: dict[tuple, Any] = {}

        self.embedding = EMBEDDINGS.build(spec.embedding.kind, runtime, **spec.embedding.params)
        self._register(self.embedding, spec.embedding.prefix)

        self.blocks = []
        for layer in spec.layers:
            position = self._position(layer.position)
            mixer = MIXERS.build(layer.mixer.kind, runtime, position, **layer.mixer.params)
            mixer_norm = NORMS.build(layer.mixer_norm.kind, runtime, **layer.mixer_norm.params)
            ff = FEED_FORWARDS.build(layer.feed_forward.kind, runtime, **layer.feed_forward.params)
            ff_norm = NORMS.build(layer.feed_forward_norm.kind, runtime, **layer.feed_forward_norm.params)
            self.blocks.append(ARRANGEMENTS.build(layer.arrangement, mixer, mixer_norm, ff, ff_norm))
            for part, part_spec in ((mixer, layer.mixer), (mixer_norm, layer.mixer_norm), (ff, layer.feed_forward),
                                    (ff_norm, layer.feed_forward_norm)):
                self._register(part, part_spec.prefix)

        self.final_norm = NORMS.build(spec.final_norm.kind, runtime, **spec.final_norm.params)
        self._register(self.final_norm, spec.final_norm.prefix)
        self.head = HEADS.build(spec.head.kind, runtime, self.embedding, **spec.head.params)
        self._register(self.head, spec.head.prefix)

        for i, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {entry.layer}; the model has {len(self.blocks)}")
        self.schedule = spec.schedule
        self.cache_plan: CachePlan = make_cache_plan(
            [self.blocks[e.layer].mixer.cache_need() for e in self.schedule], [e.cache_of for e in self.schedule])
        self.tile_specs = sorted({spec for b in self.blocks for spec in b.mixer.tile_specs()})

    # ---- construction helpers
    def _position(self, spec: PartSpec | None):
        if spec is None:
            return None
        key = spec.key()
        if key not in self._positions:
            self._positions[key] = POSITION_ENCODINGS.build(spec.kind, self.runtime, **spec.params)
        return self._positions[key]

    def _register(self, part: Part, prefix: str) -> None:
        for local, info in part.parameters().items():
            name = prefix + local
            if name in self._named:
                raise ValueError(f"two parts claim the tensor {name!r}")
            self._named[name] = (part, local, info)

    def named_parameters(self) -> dict[str, tuple[Part, str, ParamInfo]]:
        """Checkpoint name -> (part that takes it, the part's local name, shape and kind)."""
        return dict(self._named)

    def parts(self) -> list[Part]:
        seen, out = set(), []
        for part, _, _ in self._named.values():
            if id(part) not in seen:
                seen.add(id(part))
                out.append(part)
        return out

    def head_dims(self) -> tuple[int, ...]:
        return tuple(sorted({g.need.head_dim for g in self.cache_plan.groups}))

    # ---- the forward pass of one step
    def step(self, ctx: StepContext, cache) -> torch.Tensor:
        """Run the step's tokens through every scheduled block; fp32 logits ``[len(ctx.logit_rows), vocab]``."""
        x = self.embedding.forward(ctx.token_ids)
        residual = None
        for pos, entry in enumerate(self.schedule):
            block = self.blocks[entry.layer]
            # a block may leave its last projection to the next block's norm, if both sides say that they can
            after = self.blocks[self.schedule[pos + 1].layer] if pos + 1 < len(self.schedule) else None
            if getattr(block, "supports_deferred", False) and getattr(after, "accepts_deferred_input", False):
                x, residual = block.forward(x, residual, ctx, cache.layer_cache(pos, ctx), defer_output=True)
            else:
                x, residual = block.forward(x, residual, ctx, cache.layer_cache(pos, ctx))
        if ctx.logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.runtime.device)
        h = self.final_norm.forward_rows(x, residual, ctx.logit_rows)
        return self.head.forward(h)
