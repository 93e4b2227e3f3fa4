"""Weights from safetensors, by tensor name.

Like the reference's loader (oxr_runtime/weights.py:17-43) every model tensor must be assigned exactly once from
a tensor of equal shape, and names are mapped by rule (oxr_runtime/weight_names.py:25-46). Unlike it, nothing is
copied until the whole file list has been checked against the model, and a failed check raises ONE
:class:`WeightError` that lists every missing tensor, every unexpected tensor and every wrong shape. Sharded
checkpoints (``model.safetensors.index.json``) are read too.

Storage: matrices stay bfloat16 when stored so (32-bit matrices stay 32-bit), small vectors are kept in fp32;
with a float32 engine everything is widened to fp32, which is exact.
"""

from __future__ import annotations

import json
import re
from pathlib import Path

from safetensors import safe_open

from oxr_inference_b200.parts.decoder import DecoderModel


class WeightError(ValueError):
    def __init__(self, missing: list[str], unexpected: list[str], wrong: list[str], extra: list[str] | None = None):
        self.missing, self.unexpected, self.wrong_shape, self.other = missing, unexpected, wrong, extra or []
        lines = ["the checkpoint does not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
        for e in self.other:
            lines.append("  " + e)
        super().__init__("\n".join(lines))


def checkpoint_files(model_dir: str | Path) -> list[Path]:
    root = Path(model_dir)
    index = root / "model.safetensors.index.json"
    single = root / "model.safetensors"
    if single.is_file():
        return [single]
    if index.is_file():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        files = [root / n for n in names]
        absent = [str(f) for f in files if not f.is_file()]
        if absent:
            raise WeightError([], [], [], [f"shard files named by the index are absent: {absent}"])
        return files
    raise FileNotFoundError(f"{root} holds neither model.safetensors nor model.safetensors.index.json")


def load_weights(model: DecoderModel, model_dir: str | Path) -> None:
    named = model.named_parameters()
    spec = model.spec
    ignored = [re.compile(p + "$") for p in spec.ignored_tensors]
    files = checkpoint_files(model_dir)
    device = str(model.runtime.device)

    # pass 1: headers only
    plan: list[tuple[Path, str, str]] = []  # file, name in file, model name
    seen: dict[str, str] = {}
    unexpected: list[str] = []
    wrong: list[str] = []
    other: list[str] = []
    for path in files:
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():  # noqa: SIM118
                target = None
                for prefix in spec.name_prefixes:
                    if name.startswith(prefix) and name[len(prefix):] in named:
                        target = name[len(prefix):]
                        break
                if target is None:
                    bare = next((name[len(p):] for p in spec.name_prefixes if p and name.startswith(p)), name)
                    if not any(r.match(bare) for r in ignored):
                        unexpected.append(name)
                    continue
                if target in seen:
                    other.append(f"{target} is stored twice ({seen[target]} and {name})")
                    continue
                seen[target] = name
                shape = tuple(f.get_slice(name).get_shape())
                want = tuple(named[target][2].shape)
                if shape != want:
                    wrong.append(f"{name} is {list(shape)}, the model wants {list(want)}")
                    continue
                plan.append((path, name, target))
    missing = sorted(set(named) - set(seen))
    if missing or unexpected or wrong or other:
        raise WeightError(missing, sorted(unexpected), wrong, other)

    # pass 2: copy
    by_file: dict[Path, list[tuple[str, str]]] = {}
    for path, name, target in plan:
        by_file.setdefault(path, []).append((name, target))
    for path, items in by_file.items():
        with safe_open(str(path), framework="pt", device=device) as f:
            for name, target in items:
                part, local, _ = named[target]
                part.assign(local, f.get_tensor(name))
    for part in model.parts():
        part.finish_loading()
