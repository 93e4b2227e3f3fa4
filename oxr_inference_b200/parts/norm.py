"""RMSNorm with the residual add fused in."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import NORMS, DeferredLinear, Norm, ParamInfo, Runtime


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

    accepts_deferred = True

    def forward(self, x, residual, lazy: bool = False):
        """``x``: a tensor, or the part before with its last projection still to do. ``lazy``: whoever takes the result
        passes it to a product and nowhere else, so the row's scale may be left to that product."""
        if isinstance(x, DeferredLinear):
            weight = getattr(x.linear, "weight", None)
            if lazy and weight is not None:
                # a decode step: the product adds itself into the residual stream and leaves the rows' sums of squares;
                # the next part's first projection scales its sums (no norm kernel at all)
                fused = ops.linear_add(x.x, weight, residual, self.weight, self.eps)
                if fused is not None:
                    return fused
            x = x.materialize()
        return ops.add_rms_norm(x, residual, self.weight, self.eps)

    def forward_rows(self, x, residual, rows):
        if isinstance(x, DeferredLinear):
            x = x.materialize()
        return ops.add_rms_norm(x, residual, self.weight, self.eps, rows=rows)[0]
