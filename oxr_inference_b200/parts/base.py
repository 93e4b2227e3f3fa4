"""Interfaces of the parts a decoder is assembled from, their registries, and what a step hands to them.

Families and what each must provide:

* **Norm** – ``forward(x, residual) -> (normed, residual)``; the add of the not-yet-added block output into the
  fp32 residual stream is part of the norm (oxr_runtime/language.py:94-99).
* **PositionEncoding** – ``tables()``: whatever its mixers consume (rotary: fp32 cos and sin by position).
* **Mixer** – ``forward(h, ctx, cache) -> y`` over the step's packed tokens; ``cache_need()`` says what it keeps
  between steps: paged keys/values (:class:`PagedKVNeed`), fixed-size per-request state (:class:`StateNeed`),
  or nothing. ``tile_specs()`` (optional) asks the batch builder for tile lists.
* **FeedForward** – ``forward(h) -> y``.
* **Block arrangement** – puts a mixer and a feed-forward behind their norms.
* **Embedding** – ``forward(ids) -> x``; **Head** – ``forward(h) -> fp32 logits`` (it is handed the embedding part).

Every part lists its tensors with :meth:`Part.parameters` (local names; the spec's prefix makes them checkpoint
names) and receives them one by one through :meth:`Part.assign`. No part knows which model it is in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


# ------------------------------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class ParamInfo:
    shape: tuple[int, ...]
    init: str = "normal"
    """Random-weights mode: ``normal`` = N(0, std); ``around_one`` = 1 + N(0, norm_std)."""
    role: str = "matrix"
    """``matrix``: multiplied on the tensor cores, kept in the compute dtype (a tensor stored in 32-bit stays
    32-bit); ``vector``: small, used in fp32 math, always kept in fp32."""


@dataclass
class Runtime:
    """Where and how the parts run."""

    device: torch.device
    dtype: torch.dtype
    """Activation dtype: torch.bfloat16 (serving) or torch.float32 (everything in true 32-bit)."""
    max_positions: int
    status: torch.Tensor
    """Device status word that kernels write their first error to (see ``ops.check_status``)."""
    page_size: int = 16
    """Tokens per cache page (an engine setting): kernels that read the cache may plan their tiles by it."""

    def store_dtype(self, info: ParamInfo, stored: torch.dtype) -> torch.dtype:
        if info.role == "vector" or self.dtype == torch.float32:
            return torch.float32
        if stored == torch.float32:
            return torch.float32  # stored in 32-bit: stays so
        return torch.bfloat16


class Part:
    """Base of all parts: a bag of named tensors."""

    def parameters(self) -> dict[str, ParamInfo]:
        return {}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        """Take the tensor stored under local name ``name`` (host or device, dtype as stored)."""
        raise KeyError(name)

    def finish_loading(self) -> None:
        """Called once after all tensors were assigned."""


# ------------------------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token (or of the last ``window`` tokens) in pages."""

    num_kv_heads: int
    head_dim: int
    window: int = 0
    """0: all keys are kept; > 0: a query sees its last ``window`` keys, pages wholly behind that are released."""


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per request (shape without the request axis), zeroed when a request starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------------------------------- step context
@dataclass
class GroupView:
    """What one cache group looks like to a mixer during one step."""

    page_size: int
    k_pool: torch.Tensor | None
    """[layers of the group, pages, page_size, KV, D]"""
    v_pool: torch.Tensor | None
    block_table: torch.Tensor
    """int32 [requests, width]"""
    slots: torch.Tensor
    """int32 [tokens]: where each new token's K and V go (page * page_size + offset)."""
    kv_maps: object | None = None
    """TMA tensor maps over the pools (``ops.make_kv_maps``), when the sizes allow them."""


@dataclass
class LayerCache:
    """The cache of one schedule entry for this step."""

    group: GroupView | None = None
    layer_in_group: int = 0
    store: bool = True
    """False when this run reads a cache that another run fills."""
    state: torch.Tensor | None = None
    """[slots, *shape] for a mixer with :class:`StateNeed`; index with ``ctx.state_slots``."""


@dataclass
class StepContext:
    """One step's batch on the device: the new tokens of all requests packed along one axis."""

    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor      # int32 [tokens]
    positions: torch.Tensor      # int32 [tokens] absolute position of each token in its request
    req_of_token: torch.Tensor   # int32 [tokens]
    cu_q: torch.Tensor           # int32 [requests + 1]
    ctx_lens: torch.Tensor       # int32 [requests] tokens in the cache after this step
    state_slots: torch.Tensor    # int32 [requests]
    logit_rows: torch.Tensor     # int32 [wanted] indices into the token axis
    no_store_slots: torch.Tensor  # int32 [tokens], all -1
    groups: list[GroupView]
    tiles: dict[tuple[int, int, int], tuple[torch.Tensor, torch.Tensor, int]] = field(default_factory=dict)
    """(tokens per tile, fewest, most new tokens of the requests covered) -> (tile_req, tile_tok0, number of tiles)"""
    kv_len_bound: int = 0
    """No request's context is longer than this; fixed for a CUDA graph, else the step's longest context."""
    q_lens: list[int] = field(default_factory=list)       # host copies, for parts that plan on the host
    ctx_lens_host: list[int] = field(default_factory=list)
    uneven: bool = False
    """The requests' context lengths differ much (``uneven_lengths``): a mixer may then deal its work out by keys rather than by
    requests. Fixed for a captured CUDA graph (it is part of the graph's key)."""
    status: torch.Tensor | None = None
    sampling: dict[str, torch.Tensor] = field(default_factory=dict)
    """Per logit row: temperature (fp32), seed_lo, seed_hi, counter, row_slot (the row's state slot)."""

    @property
    def single_tokens(self) -> bool:
        """Every request of the step brings exactly one token (a decode step): token r is request r's, at position
        ``ctx_lens[r] - 1``."""
        return self.n_tokens == self.n_requests and all(q == 1 for q in self.q_lens)


def uneven_lengths(ctx_lens: list[int]) -> bool:
    """Whether a step's requests differ so much in length that work dealt out request by request would leave most of the GPU
    waiting for the longest: the longest is more than a quarter (and 128 keys) above the mean."""
    if len(ctx_lens) < 2:
        return False
    return max(ctx_lens) > 1.25 * (sum(ctx_lens) / len(ctx_lens)) + 128


# ------------------------------------------------------------------------------------------- families
@dataclass
class DeferredLinear:
    """The last projection of a mixer or feed-forward, not yet multiplied: ``linear(x)``. The norm that comes next may fold
    the product's add into the residual stream into the product itself. Only a norm that says ``accepts_deferred`` is
    ever handed one; anyone else who holds one calls ``materialize()``."""

    x: torch.Tensor
    linear: Callable[[torch.Tensor], torch.Tensor]
    """The projection: callable on ``x``; norms that fuse read its ``weight`` ([out, in])."""

    def materialize(self) -> torch.Tensor:
        return self.linear(self.x)


class Norm(Part):
    accepts_deferred = False
    """Whether ``forward`` takes a :class:`DeferredLinear` in place of ``x`` and a keyword ``lazy``: with ``lazy=True`` it
    may return, in place of the normalised tensor, an object that the next part's first projection normalises by itself
    (it has ``materialize()``); the block asks for that only when the part behind the norm says ``accepts_lazy_input``."""

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None):
        raise NotImplementedError

    def forward_rows(self, x: torch.Tensor, residual: torch.Tensor | None, rows: torch.Tensor) -> torch.Tensor:
        """Normalise only the given rows of ``x + residual`` (the rows whose logits are wanted)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def tables(self) -> Any:
        raise NotImplementedError


class Mixer(Part):
    accepts_lazy_input = False
    """Whether ``forward`` may be handed a lazily normalised ``h`` (it then passes ``h`` to its first projection and
    does nothing else with it)."""

    def cache_need(self) -> PagedKVNeed | StateNeed | None:
        return None

    def tile_specs(self) -> list[tuple[int, int, int]]:
        """Tile lists this mixer's kernels want from the batch builder: (tokens per tile, fewest, most new tokens of
        the requests the list covers)."""
        return []

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError

    def forward_deferred(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> "torch.Tensor | DeferredLinear":
        """``forward`` with the last projection left to the caller where the mixer ends in one (optional to override)."""
        return self.forward(h, ctx, cache)


class FeedForward(Part):
    accepts_lazy_input = False

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_deferred(self, h: torch.Tensor) -> "torch.Tensor | DeferredLinear":
        """``forward`` with the last projection left to the caller where the part ends in one (optional to override)."""
        return self.forward(h)


class Embedding(Part):
    """Token ids (int32 ``[tokens]``) to the first hidden states, in the runtime's activation dtype."""

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """Normalised hidden states of the wanted rows to fp32 logits ``[rows, vocab]``. A head is built with the model's
    embedding part as its second argument, so that it can share the table."""

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


# ------------------------------------------------------------------------------------------- registries
class Registry:
    def __init__(self, family: str):
        self.family = family
        self._items: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str, factory: Callable[..., Any] | None = None, *, replace: bool = False):
        def put(f):
            if kind in self._items and not replace:
                raise ValueError(f"{self.family} {kind!r} is already registered")
            self._items[kind] = f
            return f

        return put if factory is None else put(factory)

    def build(self, kind: str, *args, **kwargs):
        if kind not in self._items:
            raise KeyError(f"no {self.family} named {kind!r}; registered: {sorted(self._items)}")
        return self._items[kind](*args, **kwargs)

    def __contains__(self, kind: str) -> bool:
        return kind in self._items

    def kinds(self) -> list[str]:
        return sorted(self._items)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
ARRANGEMENTS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
