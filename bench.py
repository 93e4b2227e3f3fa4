#!/usr/bin/env python3
"""Measures the engine on one B200: Qwen3-8B layer sizes, bf16, random weights, synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 with 2,048 tokens of context per request,
timed on the device over K replays of the decode step; ``e2e`` is the same through ``Engine.step`` (host token ids
in through pinned memory, sampled token ids out, every step). ``prefill`` is one 2,048-token prompt in one step;
``points`` holds decode at batch 1 and 64, at longer contexts and for 32 requests of very different lengths, a longer prefill
and the two serving workloads; ``roofline`` divides the bytes a decode step has to read (every weight
once, plus the cache of the live requests) by its time. A step's inputs (15 GB of weights) are far larger than L2,
so nothing is cached between timed iterations.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096, "intermediate_size": 12288,
    "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "vocab_size": 151936, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 2560, "intermediate_size": 9728,
    "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "vocab_size": 151936, "tie_word_embeddings": True, "max_position_embeddings": 4096,
}
QWEN3_32B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 5120, "intermediate_size": 25600,
    "num_hidden_layers": 64, "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "vocab_size": 151936, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
CONTEXT = 2048
PREFILL_TOKENS = 2048
LONG_CONTEXTS = (8192, 32768)      # further decode points at batch 8
LONG_PREFILL_TOKENS = 8192         # a further prefill point
UNEVEN_CONTEXTS = [256 + round(i * (8192 - 256) / 31) for i in range(32)]   # a decode point with requests of very different lengths
METRIC = "Qwen3-8B bf16 decode tok/s at batch 8 (context 2048)"


def peaks() -> tuple[float, float, str]:
    """(HBM GB/s, bf16 TFLOP/s, 'measured' | 'fallback')"""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            p = json.loads(path.read_text())
            return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
        except (KeyError, ValueError):
            pass
    return 6650.0, 1590.0, "fallback"


def sustained_tflops() -> float | None:
    """The measured bf16 throughput of a seconds-long loop under the power cap, if the peaks file has it: the figure
    for a product timed inside a long step."""
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["bf16_tflops_sustained"])
    except (OSError, KeyError, ValueError, TypeError):
        return None


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait(timeout=10)
        self.thread.join(timeout=5)
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def reference_arm(args) -> int:
    """The unmodified reference's language path at the same config (see baseline/reference_arm.py); nothing of this
    repository's package is imported on this path."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm
    return arm.run(args, QWEN3_8B, args.context, PREFILL_TOKENS, METRIC.replace(str(CONTEXT), str(args.context)), peaks, ClockSampler)


def serving_workload(which: str) -> int:
    """The two serving workloads beside the headline: many requests through ``Engine.generate`` (wall clock, host in the
    loop). ``continuous``: Qwen3-4B sizes (tied head), 256 requests, prompts of 64..2048 and outputs of 32..512 tokens,
    greedy. ``chunked``: Qwen3-32B sizes, 32 requests of 4,096 prompt tokens cut into 2,048-token portions mixed with
    decoding, 256 output tokens each."""
    import random

    import torch

    from oxr_inference_b200 import ops
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.sampling import SamplingParams

    rng = random.Random(0)
    if which == "continuous":
        cfg, kv_gb, max_running, budget = QWEN3_4B, 40.0, 256, 8192
        work = [(rng.randint(64, 2048), rng.randint(32, 512)) for _ in range(256)]
    else:
        cfg, kv_gb, max_running, budget = QWEN3_32B, 40.0, 32, 2048 + 32
        work = [(4096, 256)] * 32
    V = cfg["vocab_size"]
    engine = Engine(random_config=cfg, seed=0, settings=EngineSettings(
        dtype="bfloat16", page_size=16, kv_cache_gb=kv_gb, max_running=max_running, max_step_tokens=budget, prefill_chunk=2048,
        max_positions=cfg["max_position_embeddings"], cuda_graphs=True, profile=True))
    prompts = [[rng.randrange(V) for _ in range(p)] for p, _ in work]
    params = [SamplingParams(max_tokens=o, ignore_eos=True) for _, o in work]
    engine.generate(prompts[:2], [SamplingParams(max_tokens=4, ignore_eos=True)] * 2)   # warm-up: libraries, first graphs
    before = dict(engine.counters)
    launches = ops.launch_count
    engine.profile.steps.clear()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    done = engine.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    # the engine's own per-step log: device milliseconds between two CUDA events around each step
    steps = [(st["ms"], st["tokens"], st["graph"], st["held"]) for st in engine.profile.steps]
    out_tokens = sum(len(c.token_ids) for c in done)
    in_tokens = sum(len(p) for p in prompts)
    assert all(len(c.token_ids) == o for c, (_, o) in zip(done, work))

    def percentiles(values, marks=(50, 90, 99)):
        v = sorted(values)
        return {f"p{q}": round(v[min(len(v) - 1, len(v) * q // 100)], 3) for q in marks} if v else {}

    h, layers, inter = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["intermediate_size"]
    heads, kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_params = h * (heads + 2 * kv) * d + heads * d * h + 3 * h * inter
    weight_bytes = 2 * (layers * layer_params + V * h)           # every matrix a decode step reads, the head included
    kv_bytes_per_token = 2 * 2 * layers * kv * d
    hbm_gbs, bf16_tflops, source = peaks()
    decode = [(ms, n, held) for ms, n, graph, held in steps if graph]
    mixed = [(ms, n) for ms, n, graph, held in steps if not graph]
    decode_fracs = [(weight_bytes + kv_bytes_per_token * held) / (ms * 1e-3) / 1e9 / hbm_gbs for ms, n, held in decode]
    mixed_flops = [2 * n * (layers * layer_params) / (ms * 1e-3) / 1e12 / bf16_tflops for ms, n in mixed if n >= 1024]
    print(json.dumps({
        "workload": which, "model": "Qwen3-4B shape (tied)" if which == "continuous" else "Qwen3-32B shape", "requests": len(work),
        "prompt_tokens": in_tokens, "output_tokens": out_tokens, "seconds": round(seconds, 3),
        "output_tok_s": round(out_tokens / seconds, 1), "total_tok_s": round((in_tokens + out_tokens) / seconds, 1),
        "steps": engine.counters["steps"] - before["steps"], "graph_steps": engine.counters["graph_steps"] - before["graph_steps"],
        "decode_step_ms": percentiles([ms for ms, _, _ in decode]), "mixed_step_ms": percentiles([ms for ms, _ in mixed]),
        "decode_step_hbm_frac": percentiles(decode_fracs, (10, 50, 90)), "mixed_step_gemm_frac": percentiles(mixed_flops, (10, 50, 90)),
        "slowest_steps_ms": [round(ms, 1) for ms, *_ in sorted(steps, reverse=True)[:4]],
        "weight_gb_per_decode_step": round(weight_bytes / 1e9, 2), "peaks": source,
        "stages": engine.profile.summary(),
        "preemptions": engine.preemptions, "gpu_launches": ops.launch_count - launches, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"], help="fewer layers than the model has (named in config)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the further points (quick runs)")
    ap.add_argument("--skip-serving", action="store_true", help="leave the two serving workloads out of `points`")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds when the decode steps are timed")
    ap.add_argument("--workload", default="decode", choices=("decode", "continuous", "chunked"),
                    help="decode: the headline line (default); continuous / chunked: the two serving workloads, one line each")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload != "decode":
        return serving_workload(args.workload)
    K, W = args.steps, max(args.warmup, 3)

    import torch

    from oxr_inference_b200 import ops
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.engine.batch import StepEntry
    from oxr_inference_b200.sampling import SamplingParams

    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    page = 16
    context = args.context
    kv_per_token = 2 * 2 * args.layers * cfg["num_key_value_heads"] * cfg["head_dim"]
    # batch 1 and 64 ride along where 64 requests of this context fit beside the weights (they do at 2,048 tokens)
    batches = (8,) if args.skip_points or 64 * context * kv_per_token > 100e9 else (8, 1, 64)
    # further points: batch 8 at longer contexts, and a longer prompt
    long_contexts = () if args.skip_points else LONG_CONTEXTS
    long_prefill = 0 if args.skip_points else LONG_PREFILL_TOKENS
    spare = 2 * (K + W) + 64
    pages = max([max(batches) * ((context + spare) // page + 2)] + [8 * ((c + spare) // page + 2) for c in long_contexts] +
                ([sum((c + spare) // page + 2 for c in UNEVEN_CONTEXTS)] if long_contexts else [])) + 64
    engine = Engine(random_config=cfg, seed=0, settings=EngineSettings(
        dtype="bfloat16", page_size=page, num_pages=pages, max_running=64, max_step_tokens=8192, prefill_chunk=2048,
        max_positions=max([4096, context + spare + 64, long_prefill + 64] + [c + spare + 64 for c in long_contexts]), cuda_graphs=True))
    model = engine.runner.model
    gen = torch.Generator().manual_seed(0)
    hbm_gbs, bf16_tflops, peak_kind = peaks()

    L, h, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, KV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_params = (H + 2 * KV) * D * h + H * D * h + 2 * I * h + I * h
    weight_bytes = 2 * (L * layer_params + V * h) + 4 * (L * (2 * h + 2 * D) + h)
    kv_bytes_per_token = 2 * L * KV * D * 2

    def fill(batch: int, budget: int, tokens) -> None:
        """`batch` requests, each with `tokens` tokens (one number, or one for each) in the cache and one token left to decode."""
        for r in list(engine.scheduler.running) + list(engine.scheduler.waiting):
            r.cancelled = True
        engine.step()
        for i in range(batch):
            p = torch.randint(0, V, (tokens if isinstance(tokens, int) else tokens[i],), generator=gen).tolist()
            engine.add_request(p, SamplingParams(max_tokens=budget, ignore_eos=True))
        while engine.scheduler.waiting or any(r.pending > 1 for r in engine.scheduler.running):
            engine.step()
        assert len(engine.scheduler.running) == batch

    def decode_device(batch: int, tokens=context) -> tuple[float, int, int]:
        """ms per decode step on the device (K replays after W), kernels per step, context length (of the first request)."""
        fill(batch, 2 * (K + W) + 8, tokens)
        plan = engine.scheduler.schedule()
        assert plan.decode_only and len(plan.entries) == batch
        entries = [StepEntry(p.request.cache, p.request.tokens[p.start:p.start + 1], [0], counter=len(p.request.output))
                   for p in plan.entries]
        tokens, _ = engine.graphs.run(entries)  # captures at first use, fills the static inputs
        key = engine.graphs.last_key
        graph = engine.graphs._graphs[key][0]
        for _ in range(W):
            graph.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(K):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / K
        ctx = plan.entries[0].start + 1
        engine.scheduler.commit(plan, {p.request.id: t for p, t in zip(plan.entries, tokens.tolist())})
        return ms, engine.graphs.kernels_per_replay[key], ctx

    sampler = ClockSampler()
    sampler.start()

    # ---- headline: batch 8, device-timed
    ms8, kernels_per_step, ctx8 = decode_device(8)
    value = 8 * 1000.0 / ms8
    step_bytes = weight_bytes + 8 * ctx8 * kv_bytes_per_token + 8 * h * 2
    achieved = step_bytes / (ms8 * 1e-3) / 1e9

    # ---- the same through the entry point: host tokens in, sampled tokens out, every step
    for _ in range(W):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e = 8 * K / e2e_s
    layout_words = next(v[1].total for k, v in engine.graphs._graphs.items() if k[0] == 8)

    points = {}
    for b in batches[1:]:
        ms, _, ctx = decode_device(b)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
        points[f"decode_b{b}_hbm_frac"] = round((weight_bytes + b * ctx * kv_bytes_per_token) / (ms * 1e-3) / 1e9 / hbm_gbs, 4)
    for c in long_contexts:
        ms, _, ctx = decode_device(8, c)
        points[f"decode_b8_ctx{c}"] = round(8 * 1000.0 / ms, 1)
        points[f"decode_b8_ctx{c}_hbm_frac"] = round((weight_bytes + 8 * ctx * kv_bytes_per_token) / (ms * 1e-3) / 1e9 / hbm_gbs, 4)

    if long_contexts:
        # requests of very different lengths, as a serving engine has them: 32 contexts evenly spaced from 256 to 8,192 tokens
        lens = UNEVEN_CONTEXTS
        ms, _, _ = decode_device(32, lens)
        points["decode_b32_ctx256_to_8192"] = round(32 * 1000.0 / ms, 1)
        points["decode_b32_ctx256_to_8192_hbm_frac"] = round((weight_bytes + (sum(lens) + 32) * kv_bytes_per_token) / (ms * 1e-3) / 1e9 / hbm_gbs, 4)

    # ---- prefill: one prompt in one step
    for r in list(engine.scheduler.running):
        r.cancelled = True
    engine.step()

    def prefill_ms_of(T: int) -> float:
        ids = torch.randint(0, V, (T,), generator=gen).tolist()
        times = []
        for i in range(W + 5):
            rc = engine.runner.cache.open("prefill")
            assert engine.runner.cache.reserve(rc, T)
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.step([StepEntry(rc, ids, [T - 1])])
            end.record()
            torch.cuda.synchronize()
            if i >= W:
                times.append(start.elapsed_time(end))
            engine.runner.cache.close(rc)
        engine.runner.check()
        return statistics.median(times)

    T = PREFILL_TOKENS
    prefill_ms = prefill_ms_of(T)
    # the fraction counts the matrix products alone (attention's flops are named beside it, not added to it)
    flops = 2 * T * L * layer_params + 2 * V * h
    attn_flops = L * 2 * H * D * T * (T + 1)
    prefill_frac = flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12)
    if long_prefill:
        ms = prefill_ms_of(long_prefill)
        points[f"prefill_{long_prefill}"] = round(long_prefill / (ms * 1e-3), 1)
        points[f"prefill_{long_prefill}_gemm_frac"] = round((2 * long_prefill * L * layer_params + 2 * V * h) / (ms * 1e-3) / (bf16_tflops * 1e12), 4)

    clocks = sampler.stop()
    launches_of_step = kernels_per_step * K
    if not (args.skip_points or args.skip_serving):
        # the two serving workloads, each in a process of its own once this one's model is gone
        del engine, model
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for which in ("continuous", "chunked"):
            try:
                res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", which], capture_output=True, text=True, timeout=900)
                line = json.loads(res.stdout.strip().splitlines()[-1])
                points[f"{which}_output_tok_s"] = line["output_tok_s"]
                points[f"{which}_decode_hbm_frac_p50"] = line["decode_step_hbm_frac"].get("p50")
                points[f"{which}_mixed_gemm_frac_p50"] = line["mixed_step_gemm_frac"].get("p50")
            except Exception as exc:   # a serving workload that fails does not take the headline with it
                points[f"{which}_error"] = f"{type(exc).__name__}: {exc}"[:200]
    out = {
        "metric": METRIC.replace(str(CONTEXT), str(context)), "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_of_model": QWEN3_8B["num_hidden_layers"], "hidden": h,
                   "heads": H, "kv_heads": KV, "head_dim": D, "intermediate": I, "vocab": V, "global_batch": 8,
                   "seq_len": context, "page_size": page, "tied": False, "parallelism": "single GPU",
                   "l2": "step inputs (15 GB of weights) exceed L2", "peaks": peak_kind},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": layout_words * 4, "d2h_bytes_per_step": (8 + 2) * 4},
        "gpu_launches": launches_of_step,
        "prefill": {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4),
                    "attention_tflops_in_step": round(attn_flops / 1e12, 3),
                    **({"frac_of_sustained": round(flops / (prefill_ms * 1e-3) / (sustained_tflops() * 1e12), 4)} if sustained_tflops() else {})},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
