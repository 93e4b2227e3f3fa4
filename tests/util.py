"""Shared by the tests: the two tiny configurations, model folders, the replay driver, comparisons."""

from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent

# Two tiny Qwen3 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 64, "intermediate_size": 128,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "vocab_size": 256, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "eos_token_id": 255,
}  # head_dim absent: 64 / 4 = 16; page 16
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 96, "intermediate_size": 160,
    "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0, "vocab_size": 509, "tie_word_embeddings": False, "max_position_embeddings": 384,
    "use_sliding_window": True, "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"], "eos_token_id": [507, 508],
}  # GQA ratio 3, heads * head_dim != hidden, odd vocabulary, a windowed layer; page 8
PAGE = {"A": 16, "B": 8}
CONFIGS = {"A": TINY_A, "B": TINY_B}


def make_folder(tmp: Path, name: str, seed: int = 0, dtype: str = "bfloat16", sharpen: float = 2.0) -> Path:
    """A model folder with random weights. The q/k head-norm weights are scaled by ``sharpen`` so that attention is
    peaked: with near-uniform attention a lost or doubled key would change the logits too little to see."""
    from safetensors.torch import load_file, save_file

    from oxr_inference_b200.weights import write_random_model

    folder = write_random_model(CONFIGS[name], tmp / f"tiny_{name}_{dtype}_{seed}", seed, dtype=dtype)
    if sharpen != 1.0:
        path = folder / "model.safetensors"
        tensors = load_file(str(path))
        for k in tensors:
            if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
                tensors[k] = (tensors[k].float() * sharpen ** 0.5).to(tensors[k].dtype)
        save_file(tensors, str(path), metadata={"format": "pt"})
    return folder


def token_ids(name: str, n: int, seed: int) -> list[int]:
    rng = random.Random(seed * 7919 + n)
    return [rng.randrange(CONFIGS[name]["vocab_size"]) for _ in range(n)]


_plain_cache: dict = {}


def plain_logits(folder: Path, ids: list[int]) -> torch.Tensor:
    """fp32 logits of the whole sequence from the plain implementation (cached per folder and sequence)."""
    from plain import qwen3_plain as QP

    key = (str(folder), tuple(ids))
    if key not in _plain_cache:
        cfg, w = QP.read_model(folder, torch.float32)
        _plain_cache[key] = QP.logits(cfg, w, ids)
    return _plain_cache[key]


OBSERVED: dict[str, list[float]] = {}
"""Largest bfloat16 errors seen per test (rms of rms, largest of scale); written as JSON to the file that the
environment variable OXR_TEST_ERRORS names, when it is set, as the process ends."""


def _record(rms: float, worst: float) -> None:
    import atexit
    import os

    if not OBSERVED and os.environ.get("OXR_TEST_ERRORS"):
        atexit.register(lambda: Path(os.environ["OXR_TEST_ERRORS"]).write_text(json.dumps(OBSERVED, indent=1)))
    key = os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0]
    seen = OBSERVED.setdefault(key, [0.0, 0.0])
    seen[0], seen[1] = max(seen[0], rms), max(seen[1], worst)


def compare(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32: 1e-4 of the logits' scale, absolute and relative. bfloat16: rms error <= 3e-2 of the rms, largest
    error <= 5e-2 of the largest logit. Observed on a B200 over all cuttings: at most 1.7e-2 / 2.4e-2 on the tiny
    configurations and the odd sizes, 2.5e-2 / 2.7e-2 on four layers of Qwen3-8B's sizes with sharpened attention."""
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = want.abs().max().item()
    err = (got - want).abs()
    if dtype == "float32":
        bad = err > 1e-4 * scale + 1e-4 * want.abs()
        assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.numel()} logits off by more than 1e-4; worst {err.max().item():.3e} "
                               f"(scale {scale:.3e}) at row {int(err.max(1).values.argmax())}")
    else:
        rms = (err.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item()
        worst_row = int(err.max(1).values.argmax())
        _record(rms, err.max().item() / scale)
        assert rms <= 3e-2 and err.max().item() <= 5e-2 * scale, (
            f"{what}: rms error {rms:.3e} of rms, largest {err.max().item() / scale:.3e} of scale, at row {worst_row}")


class Replay:
    """Drives ``bin/trace_run`` over a pipe: send a step, wait for its ``done`` line, read its logits file."""

    def __init__(self, folder: Path, dtype: str, out: Path, max_tokens: int, page_size: int = 16, env: dict | None = None):
        self.out = out
        self.vocab = json.loads((folder / "config.json").read_text())["vocab_size"]
        cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
               "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.n = 0

    def step(self, entries: list[dict], end: list[str] = ()) -> torch.Tensor | None:
        step = self.n
        self.n += 1
        self.proc.stdin.write(json.dumps({"step": step, "entries": entries, "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        assert line.strip() == f"done {step}", f"trace_run answered {line!r} (exit code {self.proc.poll()})"
        wanted = sum(len(e.get("want", [])) for e in entries)
        path = self.out / f"{step}.f32"
        if wanted == 0:
            assert not path.exists()
            return None
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * self.vocab, f"step {step}: {data.size} floats for {wanted} rows of {self.vocab}"
        return torch.from_numpy(data.reshape(wanted, self.vocab).copy())

    def close(self) -> int:
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        self.proc.stdout.close()
        return code
