"""Dense SiLU-gated feed-forward."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import FEED_FORWARDS, DeferredLinear, FeedForward, ParamInfo, Runtime
from oxr_inference_b200.parts.linear import StackedLinear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``down( silu(h W_gate^T) * (h W_up^T) )`` with gate and up as one product (oxr_runtime/language.py:266-269,
    102-104). No biases (language.py:229-231)."""

    def __init__(self, runtime: Runtime, *, hidden_size: int, intermediate_size: int):
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        # gate and up rows alternate in groups of 8 where the size allows: the decode kernel then holds a gate and its
        # up in one block and applies SiLU in its epilogue
        self.gate_up = StackedLinear(runtime, self.hidden, {"gate_proj.weight": self.inter, "up_proj.weight": self.inter},
                                     interleave=ops.GATE_UP_INTERLEAVE)
        self.down = StackedLinear(runtime, self.inter, {"down_proj.weight": self.hidden})

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.gate_up.parameters(), **self.down.parameters()}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.gate_up.outs:
            self.gate_up.assign(name, tensor)
        elif name in self.down.outs:
            self.down.assign(name, tensor)
        else:
            raise KeyError(name)

    accepts_lazy_input = True   # h goes into the gate|up projection and nowhere else

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(self._gated(h))

    def forward_deferred(self, h: torch.Tensor) -> DeferredLinear:
        return DeferredLinear(self._gated(h), self.down)

    def _gated(self, h: torch.Tensor) -> torch.Tensor:
        return ops.gated_silu_linear(h, self.gate_up.weight, self.gate_up.interleave)
