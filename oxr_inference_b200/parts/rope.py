"""Rotary position encoding, half-split (GPT-NeoX) form."""

from __future__ import annotations

import torch

from oxr_inference_b200.parts.base import POSITION_ENCODINGS, PositionEncoding, Runtime


@POSITION_ENCODINGS.register("rope_neox")
class RotaryTable(PositionEncoding):
    """fp32 ``cos`` and ``sin`` of ``position * theta^(-2i/dim)`` for i < dim/2, one row per position.

    Built exactly as the reference builds it: fp32 ``inv_freq``, fp32 outer product, then cos/sin
    (oxr_runtime/language.py:160-165). The reference then rounds the table to the model dtype
    (language.py:167-170); here the angles stay fp32 whatever the activation dtype. The table is computed on the
    host so that it does not depend on the device's math library, then copied once.
    """

    def __init__(self, runtime: Runtime, *, dim: int, theta: float):
        if dim % 2:
            raise ValueError(f"rotary dimension {dim} is odd")
        self.dim, self.theta = int(dim), float(theta)
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float) / self.dim))
        freqs = torch.outer(torch.arange(runtime.max_positions, dtype=torch.float), inv_freq)
        self.cos = freqs.cos().to(runtime.device).contiguous()
        self.sin = freqs.sin().to(runtime.device).contiguous()

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin
