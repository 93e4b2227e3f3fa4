"""Engine settings: what is chosen at start-up rather than read from the model folder.

Names follow the reference's ``EngineSettings`` (oxr_runtime/engine.py:107-127) where it has them:
``kv_cache_gb``, ``max_running``, ``max_positions``, ``cuda_graphs``, ``max_waiting``. The reference's
``max_prefill_tokens`` bounds a batch of whole prompts; here prompts are cut into portions, so the bound is
the token budget of one step (``max_step_tokens``) and the largest portion (``prefill_chunk``).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineSettings:
    kv_cache_gb: float = 16.0
    """Device memory for the paged cache; ignored when ``num_pages`` is given."""
    num_pages: int | None = None
    """Pages per cache group (overrides ``kv_cache_gb``)."""
    page_size: int = 16
    max_running: int = 256
    """Most requests that hold cache pages at one time."""
    max_waiting: int = 2048
    """Most queued requests; beyond it ``add_request`` raises ``Busy`` (oxr_runtime/engine.py:367-368)."""
    max_step_tokens: int = 8192
    """Token budget of one step: decode tokens first, the rest goes to prompt portions."""
    prefill_chunk: int = 2048
    """Largest portion of one prompt in one step."""
    max_positions: int | None = None
    """Longest sequence (prompt + output); None takes ``max_position_embeddings`` of the model."""
    cuda_graphs: bool = True
    """Replay decode-only steps from CUDA graphs (oxr_runtime/decode_graph.py)."""
    dtype: str = "bfloat16"
    """``bfloat16``: the serving kernels; ``float32``: every operation in true 32-bit."""
    profile: bool = False
    """Keep per-stage timers and a per-step log in ``Engine.profile`` (also switched on by ``OXR_PROFILE=1`` in the
    environment, the reference's switch, oxr_runtime/engine.py:62-63)."""
    step_tile: int | None = None
    """Rows of the widest tile of the kernels that run a step; the scheduler trims prompt portions so that a step's
    tokens come to whole tile rows. None asks the kernels (``ops.STEP_TILE_ROWS``), 0 turns the trimming off."""

    def __post_init__(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.max_step_tokens < 1 or self.prefill_chunk < 1 or self.max_running < 1:
            raise ValueError("max_step_tokens, prefill_chunk and max_running must be at least 1")
