"""Per-request sampling options and the result of a request."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 16
    """Most tokens to generate (the reference's per-request ``max_tokens``, oxr_runtime/engine.py:343-371)."""
    temperature: float = 0.0
    """0: greedy, the first maximum of the fp32 logits (all the reference does, oxr_runtime/decode_graph.py:82);
    > 0: a draw from softmax(logits / temperature)."""
    seed: int = 0
    """Seed of the request's draws; draw i depends on (seed, i) only."""
    repetition_penalty: float = 1.0
    """vLLM-style penalty on tokens already seen, prompt included (oxr_runtime/engine.py:632-639); 1 = off."""
    ignore_eos: bool = False
    """Keep generating past an end-of-sequence token (for measurements with random weights)."""
    stop_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if not 0 <= self.seed < (1 << 64):
            raise ValueError("seed must fit 64 bits")


@dataclass
class Completion:
    """What a finished request returns (oxr_runtime/engine.py:130-137)."""

    token_ids: list[int]
    finish_reason: str
    """``stop`` (end-of-sequence or stop token, not included), ``length`` (max_tokens, the position limit, or a
    request larger than the whole cache)."""
    prompt_tokens: int
    seconds: float
    text: str | None = None
    preemptions: int = 0
    request_id: int = field(default=-1)
