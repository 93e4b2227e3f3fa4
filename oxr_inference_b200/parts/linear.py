"""Weight matrices of linear maps, possibly several checkpoint tensors stacked into one product."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import ParamInfo, Runtime


class StackedLinear:
    """``y = x @ W.T`` where ``W [sum(out_i), in]`` is filled row range by row range from separate checkpoint
    tensors. The reference concatenates q|k|v and gate|up after loading (oxr_runtime/language.py:234-245); here
    each tensor is copied straight into its rows of one buffer, so no second copy of the weights ever exists."""

    def __init__(self, runtime: Runtime, in_features: int, outs: dict[str, int]):
        self.runtime, self.in_features = runtime, int(in_features)
        self.outs = {k: int(v) for k, v in outs.items()}
        self.offsets: dict[str, int] = {}
        row = 0
        for name, n in self.outs.items():
            self.offsets[name] = row
            row += n
        self.out_features = row
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {name: ParamInfo((n, self.in_features)) for name, n in self.outs.items()}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        info = self.parameters()[name]
        if self.weight is None:
            dtype = self.runtime.store_dtype(info, tensor.dtype)
            self.weight = torch.empty((self.out_features, self.in_features), dtype=dtype, device=self.runtime.device)
        lo = self.offsets[name]
        self.weight[lo:lo + self.outs[name]].copy_(tensor)

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype)
