"""The reference arm of bench.py: NickWilde18/oxr-inference's own language path, unmodified, at the bench's config.

What runs is the reference's stock code from ``baseline/_ref/oxr_runtime`` (a plain copy of its package; it has no
setup.py or pyproject.toml, so pip cannot install it): ``LanguageModel`` with ``fuse_projections`` and ``cast_rope``
(language.py:149-214), its ``KVCache`` with its own page size of 256 (kv_cache.py:22-52), prompts through
``LanguageModel.prefill`` the way ``Engine._prefill_batch`` calls it (engine.py:523-555), decoding through
``DecodeGraphs.run`` (decode_graph.py:92-119: the captured step with embedding and argmax that its engine replays,
engine.py:579-590), attention through its default backend (flash-attn 2, attention.py:31-42) and its Triton kernel
for q/k norm, rotation and the cache store (kernels.py:66-99). Its ``Engine`` class is not used: it only loads the
vision+language folder of its own model (engine.py:208-215). Nothing of this repository's package is imported here.

Timing is the same as in the other arm: ``value`` from CUDA events around K replays of the batch-8 decode graph after
W, ``e2e`` from K calls of ``DecodeGraphs.run`` with host lists in and ``tokens.tolist()`` out (what
``Engine._decode`` and ``_emit`` do per step), ``prefill`` from one 2,048-token ``prefill`` call with the logits of
its last token, points at batch 1 and 64.
"""

from __future__ import annotations

import json
import os
import shutil
import statistics
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def _ensure_copy() -> str | None:
    """The reference's package under baseline/_ref; copied from the mounted reference tree if it is not there yet."""
    if (REF / "oxr_runtime" / "language.py").is_file():
        return None
    for src in (Path(os.environ.get("OXR_REFERENCE_TREE", "/root/reference")) / "oxr_runtime",):
        if (src / "language.py").is_file():
            REF.mkdir(parents=True, exist_ok=True)
            shutil.copytree(src, REF / "oxr_runtime", dirs_exist_ok=True)
            return None
    return "baseline/_ref/oxr_runtime is missing and no reference tree is mounted to copy it from"


def run(args, model_cfg: dict, context: int, prefill_tokens: int, metric: str, peaks, clock_sampler) -> int:
    why = _ensure_copy()
    if why:
        return _unavailable(why)
    sys.path.insert(0, str(REF))
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device here: the reference's language path needs a GPU (flash-attn 2, Triton)")
        from oxr_runtime.config import LanguageConfig
        from oxr_runtime.decode_graph import DecodeGraphs
        from oxr_runtime.kv_cache import BLOCK_SIZE, KVCache, blocks_for
        from oxr_runtime.language import LanguageModel, PrefillBatch, slot_of
        from oxr_runtime import attention as ref_attention
    except Exception as exc:  # an import error of flash-attn or triton is the finding; quote it
        return _unavailable(f"importing the reference's language path failed: {type(exc).__name__}: {exc}")

    K, W = args.steps, max(args.warmup, 3)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    dtype = torch.bfloat16
    L = args.layers
    cfg = LanguageConfig(
        hidden_size=model_cfg["hidden_size"], intermediate_size=model_cfg["intermediate_size"], num_layers=L,
        num_heads=model_cfg["num_attention_heads"], num_kv_heads=model_cfg["num_key_value_heads"],
        head_dim=model_cfg["head_dim"], rms_norm_eps=model_cfg["rms_norm_eps"], rope_theta=model_cfg["rope_theta"],
        vocab_size=model_cfg["vocab_size"])
    h, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    H, KV, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    batches = (8,) if args.skip_points else (8, 1, 64)
    max_positions = max(4096, context + 2 * (K + W) + 128)

    try:
        torch.manual_seed(0)
        with torch.device(dev):
            model = LanguageModel(cfg, max_positions).to(dtype)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
                    p.fill_(1.0)
                else:
                    p.normal_(0.0, 0.02)
        model.cast_rope(dtype)
        model.fuse_projections()
        model = model.eval().requires_grad_(False)

        per_request = blocks_for(context + 2 * (K + W) + 64)
        cache = KVCache(cfg, max(batches) * per_request + 8, dtype=dtype, device=dev)
        stream = torch.cuda.Stream(device=dev, priority=-1)
        with torch.inference_mode():
            graphs = DecodeGraphs(model, cache, max_batch=max(batches), max_positions=max_positions, stream=stream)
        gen = torch.Generator().manual_seed(0)

        def prefill(prompts: list[list[int]], tables: list[list[int]]) -> list[int]:
            """One prefill call over whole prompts, as Engine._prefill_batch issues it; returns the greedy first tokens."""
            import numpy as np
            lengths = [len(p) for p in prompts]
            local = [np.arange(n) for n in lengths]
            ids = torch.from_numpy(np.concatenate([np.asarray(p) for p in prompts])).to(dev)
            positions = torch.from_numpy(np.concatenate(local)).to(dev)
            slots = torch.from_numpy(np.concatenate([
                np.asarray(blocks)[p // BLOCK_SIZE] * BLOCK_SIZE + p % BLOCK_SIZE for blocks, p in zip(tables, local)])).to(dev)
            cu = torch.tensor([0, *np.cumsum(lengths)], device=dev, dtype=torch.int32)
            with torch.inference_mode():
                hidden = model.prefill(PrefillBatch(model.embed_tokens(ids), positions, cu, max(lengths), slots), cache)
                logits = model.logits(hidden[cu[1:].long() - 1])
                return logits.argmax(dim=-1).tolist()

        class Live:
            def __init__(self, batch: int):
                self.tables = []
                for _ in range(batch):
                    blocks = cache.allocate(blocks_for(context + 1))
                    assert blocks is not None
                    self.tables.append(blocks)
                self.lengths = [context] * batch
                self.last = []
                for i in range(0, batch, 8):
                    prompts = [torch.randint(0, V, (context,), generator=gen).tolist() for _ in self.tables[i:i + 8]]
                    self.last += prefill(prompts, self.tables[i:i + 8])

            def step_inputs(self):
                for blocks, n in zip(self.tables, self.lengths):
                    if n + 1 > len(blocks) * BLOCK_SIZE:      # Engine._grow
                        more = cache.allocate(1)
                        assert more is not None
                        blocks.extend(more)
                return (self.last, list(self.lengths), [slot_of(b, n) for b, n in zip(self.tables, self.lengths)],
                        [n + 1 for n in self.lengths], self.tables)

            def step(self) -> None:
                """What Engine._decode and _emit do for a step whose requests all go on."""
                with torch.inference_mode(), torch.cuda.stream(stream):
                    _, tokens = graphs.run(*self.step_inputs())
                    self.last = tokens.tolist()
                self.lengths = [n + 1 for n in self.lengths]

            def close(self) -> None:
                for blocks in self.tables:
                    cache.release(blocks)

        def decode_device(batch: int):
            live = Live(batch)
            live.step()                                       # fills the graph's static inputs
            bucket = next(b for b in graphs.buckets if b >= batch)
            graph = graphs._graphs[bucket][0]
            with torch.cuda.stream(stream):
                for _ in range(W):
                    graph.replay()
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                for _ in range(K):
                    graph.replay()
                end.record()
                torch.cuda.synchronize()
            return start.elapsed_time(end) / K, live

        sampler = clock_sampler()
        sampler.start()
        ms8, live = decode_device(8)
        ctx8 = live.lengths[0]
        for _ in range(W):
            live.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(K):
            live.step()
        torch.cuda.synchronize()
        e2e = 8 * K / (time.perf_counter() - t0)
        h2d = sum(dst[:8].numel() * dst.element_size() for dst, _ in graphs._staging)
        live.close()

        points = {}
        for b in batches[1:]:
            ms, lv = decode_device(b)
            points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
            lv.close()

        T = prefill_tokens
        ids = torch.randint(0, V, (T,), generator=gen).tolist()
        times = []
        for i in range(W + 5):
            blocks = cache.allocate(blocks_for(T + 1))
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            prefill([ids], [blocks])
            end.record()
            torch.cuda.synchronize()
            if i >= W:
                times.append(start.elapsed_time(end))
            cache.release(blocks)
        prefill_ms = statistics.median(times)
        clocks = sampler.stop()
    except Exception as exc:
        import traceback
        traceback.print_exc(file=sys.stderr)
        return _unavailable(f"the reference's language path failed on this GPU: {type(exc).__name__}: {exc}")

    hbm_gbs, bf16_tflops, peak_kind = peaks()
    layer_params = (H + 2 * KV) * D * h + H * D * h + 2 * I * h + I * h
    weight_bytes = 2 * (L * layer_params + V * h) + 2 * (L * (2 * h + 2 * D) + h)
    kv_bytes_per_token = 2 * L * KV * D * 2
    step_bytes = weight_bytes + 8 * ctx8 * kv_bytes_per_token + 8 * h * 2
    achieved = step_bytes / (ms8 * 1e-3) / 1e9
    gemm_flops = 2 * T * L * layer_params + 2 * V * h
    attn_flops = L * 2 * H * D * T * (T + 1)
    print(json.dumps({
        "metric": metric, "value": round(8 * 1000.0 / ms8, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)", "impl": "reference",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_of_model": model_cfg["num_hidden_layers"], "hidden": h,
                   "heads": H, "kv_heads": KV, "head_dim": D, "intermediate": I, "vocab": V, "global_batch": 8,
                   "seq_len": context, "page_size": BLOCK_SIZE, "tied": False, "parallelism": "single GPU",
                   "l2": "step inputs (15 GB of weights) exceed L2", "peaks": peak_kind,
                   "attention": ref_attention.BACKEND},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 * 8},
        "prefill": {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(gemm_flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12), 4),
                    "attention_tflops_in_step": round(attn_flops / 1e12, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points, "clocks": clocks}))
    return 0
