"""Builds the model, its cache and its step function from a model folder or a configuration."""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.cache.manager import CacheManager
from oxr_inference_b200.config.model_config import read_config_json
from oxr_inference_b200.config.registry import resolve_architecture
from oxr_inference_b200.engine.batch import BatchBuilder, StepEntry
from oxr_inference_b200.parts.base import Runtime
from oxr_inference_b200.parts.decoder import DecoderModel
from oxr_inference_b200.weights.loader import load_weights
from oxr_inference_b200.weights.random_init import fill_random

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def require_cuda(device: str | torch.device = "cuda") -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this engine runs on a CUDA device only (sm_100a kernels, no CPU path); "
                           f"asked for {device}, torch.cuda.is_available() = {torch.cuda.is_available()}")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    # Matrix products of the 32-bit path and the fp32 accumulation of the 16-bit path are to be exact.
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    return device


class ModelRunner:
    """A model with its weights, its cache and its step function: what generation and trace replay both drive."""

    def __init__(self, model: DecoderModel, config: Any, *, page_size: int, num_pages: int, max_requests: int):
        self.model, self.config = model, config
        rt = model.runtime
        if rt.page_size != page_size:
            raise ValueError(f"the model was built for pages of {rt.page_size} tokens, the cache is asked for {page_size}")
        ops.warm_up(model.head_dims())
        self.cache = CacheManager(model.cache_plan, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                                  device=rt.device, dtype=rt.dtype)
        self.builder = BatchBuilder(self.cache, model.tile_specs, rt.device, rt.status)
        self.steps = 0

    # ---- construction
    @staticmethod
    def build_model(raw_config: Mapping[str, Any], generation: Mapping[str, Any] | None, *, dtype: str,
                    device: str | torch.device = "cuda", max_positions: int | None = None, page_size: int = 16):
        dev = require_cuda(device)
        arch = resolve_architecture(raw_config)
        config = arch.config_from_dict(raw_config, generation)
        spec = arch.model_spec(config)
        runtime = Runtime(device=dev, dtype=DTYPES[dtype], max_positions=max_positions or spec.max_positions,
                          status=ops.new_status(dev), page_size=page_size)
        return DecoderModel(spec, runtime), config

    @classmethod
    def from_folder(cls, model_dir: str | Path, *, dtype: str, page_size: int, num_pages: int, max_requests: int,
                    device: str | torch.device = "cuda", max_positions: int | None = None) -> "ModelRunner":
        raw, generation = read_config_json(model_dir)
        model, config = cls.build_model(raw, generation, dtype=dtype, device=device, max_positions=max_positions, page_size=page_size)
        load_weights(model, model_dir)
        return cls(model, config, page_size=page_size, num_pages=num_pages, max_requests=max_requests)

    @classmethod
    def from_config(cls, raw_config: Mapping[str, Any], seed: int, *, dtype: str, page_size: int, num_pages: int,
                    max_requests: int, device: str | torch.device = "cuda", max_positions: int | None = None,
                    std: float = 0.02, norm_std: float = 0.1) -> "ModelRunner":
        """Random weights drawn on the device (no file)."""
        model, config = cls.build_model(raw_config, None, dtype=dtype, device=device, max_positions=max_positions, page_size=page_size)
        fill_random(model, seed, std=std, norm_std=norm_std)
        return cls(model, config, page_size=page_size, num_pages=num_pages, max_requests=max_requests)

    # ---- the step function
    @torch.inference_mode()
    def step(self, entries: list[StepEntry], *, advance: bool = True) -> torch.Tensor:
        """Run one batch of (request, its next tokens): prompt portions beside single decoded tokens, cut anywhere.

        Only the given tokens are computed, against the cache earlier steps left; their keys and values are added
        to it. Pages for them must have been reserved (``cache.reserve``). Returns fp32 logits
        ``[sum(len(e.want)), vocab]`` in entry order, then ``want`` order. With ``advance`` each request's cached
        length moves forward and pages a window has passed are released."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        ctx = self.builder.build(entries)
        logits = self.model.step(ctx, self.cache)
        if advance:
            for e in entries:
                self.cache.advance(e.cache, e.cache.length + len(e.tokens))
        self.steps += 1
        return logits

    def check(self) -> None:
        """Raise if any kernel reported an error since the last check (synchronises)."""
        ops.check_status(self.model.runtime.status)
