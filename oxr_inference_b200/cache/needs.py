"""What a mixer may ask the cache to keep for it between steps."""

from __future__ import annotations

from dataclasses import dataclass

import torch

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
