"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode in its engine; its tests draw norm weights as 1 + 0.1 N(0,1) and everything else
as 0.2 N(0,1) (tests/test_language_fused.py:77-86). Here matrices and the embedding are N(0, std) and norm
weights 1 + N(0, norm_std). Each tensor's values depend on (seed, tensor name) only, not on the order of tensors.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Mapping

import torch
from safetensors.torch import save_file

from oxr_inference_b200.config.registry import resolve_architecture
from oxr_inference_b200.parts.base import ParamInfo, Runtime
from oxr_inference_b200.parts.decoder import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, info: ParamInfo, seed: int, *, std: float, norm_std: float, device: str | torch.device = "cpu",
                  dtype: torch.dtype = torch.float32) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, name))
    t = torch.randn(info.shape, generator=gen, dtype=torch.float32, device=device)
    t = 1.0 + norm_std * t if info.init == "around_one" else std * t
    return t.to(dtype)


def shape_only_model(raw_config: Mapping[str, Any]) -> DecoderModel:
    """The model's structure on the host, with no weights: enough to list tensor names and shapes."""
    arch = resolve_architecture(raw_config)
    spec = arch.model_spec(arch.config_from_dict(raw_config, None))
    cpu = torch.device("cpu")
    runtime = Runtime(device=cpu, dtype=torch.float32, max_positions=1, status=torch.zeros(4, dtype=torch.int32))
    return DecoderModel(spec, runtime)


def write_random_model(raw_config: Mapping[str, Any], out_dir: str | Path, seed: int, *, dtype: str = "bfloat16",
                       std: float = 0.02, norm_std: float = 0.1) -> Path:
    """Write ``config.json`` and ``model.safetensors`` with random weights; returns the folder."""
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    model = shape_only_model(raw_config)
    tensors = {name: random_tensor(name, info, seed, std=std, norm_std=norm_std, dtype=_DTYPES[dtype]).contiguous()
               for name, (_, _, info) in model.named_parameters().items()}
    config = dict(raw_config)
    config["torch_dtype"] = dtype
    (out / "config.json").write_text(json.dumps(config, indent=1))
    save_file(tensors, str(out / "model.safetensors"), metadata={"format": "pt"})
    return out


def fill_random(model: DecoderModel, seed: int, *, std: float = 0.02, norm_std: float = 0.1,
                stored_dtype: torch.dtype = torch.bfloat16) -> None:
    """Give ``model`` random weights in place, drawn on its device (no file): for measurements at sizes whose
    checkpoint would take minutes to write and read back."""
    device = model.runtime.device
    for name, (part, local, info) in model.named_parameters().items():
        part.assign(local, random_tensor(name, info, seed, std=std, norm_std=norm_std, device=device, dtype=stored_dtype))
    for part in model.parts():
        part.finish_loading()
