"""RMSNorm with the residual add fused in."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import NORMS, Norm, ParamInfo, Runtime


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """``out = (x + residual) * rsqrt(mean((x + residual)^2) + eps) * weight`` with the sum kept as the new fp32
    residual (oxr_runtime/language.py:69-72,94-99; layer 0 has no residual yet, language.py:253-257)."""

    def __init__(self, runtime: Runtime, *, size: int, eps: float):
        self.runtime, self.size, self.eps = runtime, int(size), float(eps)
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {"weight": ParamInfo((self.size,), init="around_one", role="vector")}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight":
            raise KeyError(name)
        self.weight = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()

    def forward(self, x, residual):
        return ops.add_rms_norm(x, residual, self.weight, self.eps)

    def forward_rows(self, x, residual, rows):
        return ops.add_rms_norm(x, residual, self.weight, self.eps, rows=rows)[0]
