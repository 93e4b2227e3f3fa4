"""Weight matrices of linear maps, possibly several checkpoint tensors stacked into one product."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import ParamInfo, Runtime


class StackedLinear:
    """``y = x @ W.T`` where ``W [sum(out_i), in]`` is filled row range by row range from separate checkpoint
    tensors. The reference concatenates q|k|v and gate|up after loading (oxr_runtime/language.py:234-245); here
    each tensor is copied straight into its rows of one buffer, so no second copy of the weights ever exists."""

    def __init__(self, runtime: Runtime, in_features: int, outs: dict[str, int], interleave: int = 0):
        """``interleave`` > 0 (two tensors of equal height, a multiple of it): rows alternate between the two tensors in
        groups of that many, rows [2 g i, 2 g i + g) from the first and the next g from the second, instead of one
        tensor after the other."""
        self.runtime, self.in_features = runtime, int(in_features)
        self.outs = {k: int(v) for k, v in outs.items()}
        heights = list(self.outs.values())
        self.interleave = int(interleave) if interleave and len(heights) == 2 and heights[0] == heights[1] and heights[0] % interleave == 0 else 0
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
        dtype = self.runtime.store_dtype(info, tensor.dtype)
        if self.weight is None:
            self.weight = torch.empty((self.out_features, self.in_features), dtype=dtype, device=self.runtime.device)
        elif dtype == torch.float32 and self.weight.dtype != torch.float32:
            # one of the stacked tensors is stored in 32-bit: the whole product is then kept and multiplied in 32-bit,
            # whichever tensor the file happens to list first
            self.weight = self.weight.float()
        if self.interleave:
            g, which = self.interleave, list(self.outs).index(name)
            self.weight.view(-1, 2, g, self.in_features)[:, which].copy_(tensor.view(-1, g, self.in_features))
            return
        lo = self.offsets[name]
        self.weight[lo:lo + self.outs[name]].copy_(tensor)

    def __call__(self, x, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """``x`` may be a lazily normalised input (``ops.NormedLazily``): the product then normalises it itself."""
        return ops.linear(x, self.weight, out_dtype)
