"""The Python entry point: ``Engine(model_dir, EngineSettings()).generate(prompts, SamplingParams())``.

The reference's engine takes a model folder and settings, accepts requests while it runs, and hands back a
``Completion`` per request (oxr_runtime/engine.py:200-384). This one is driven by the caller's thread:
``add_request`` queues, ``step`` runs one scheduler iteration (one batch through the model), ``generate`` loops
until everything queued is finished. Prompts are token ids; text goes in and out only when the model folder has a
``tokenizer.json`` (oxr_runtime/prompt.py:26-38).
"""

from __future__ import annotations

import logging
import os
import time
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.cache.manager import CacheManager
from oxr_inference_b200.config.model_config import read_config_json
from oxr_inference_b200.config.settings import EngineSettings
from oxr_inference_b200.engine.batch import StepEntry
from oxr_inference_b200.engine.graphs import DecodeGraphs
from oxr_inference_b200.engine.runtime import DTYPES, ModelRunner
from oxr_inference_b200.engine.scheduler import Busy, Request, Scheduler, StepPlan  # noqa: F401
from oxr_inference_b200.sampling.params import Completion, SamplingParams  # noqa: F401
from oxr_inference_b200.weights.loader import load_weights
from oxr_inference_b200.weights.random_init import fill_random

log = logging.getLogger(__name__)


class StageTimers:
    """Per-stage counters of the engine's step, as the reference keeps them under ``OXR_PROFILE=1``
    (oxr_runtime/engine.py:65-104: cumulative seconds and counts per stage, a ``summary()``). Host stages are wall-clock
    (``schedule``, ``build`` = filling and copying the staging block and issuing the step, ``wait`` = blocked on the
    step's one synchronisation, ``commit``); the device time of the step itself comes from two CUDA events around it
    (``decode_graph`` for a replayed decode step, ``forward`` for an eager or mixed step), read after the step's own
    synchronisation, so profiling adds no synchronisation. ``steps`` lists every step: its device milliseconds, its
    tokens, whether it was a replayed decode step, and the tokens the running requests held in the cache."""

    def __init__(self, enabled: bool):
        self.enabled = enabled
        self.seconds: dict[str, float] = {}
        self.counts: dict[str, int] = {}
        self.steps: list[dict] = []

    def add(self, name: str, seconds: float, count: int = 1) -> None:
        self.seconds[name] = self.seconds.get(name, 0.0) + seconds
        self.counts[name] = self.counts.get(name, 0) + count

    def summary(self) -> dict[str, dict[str, float]]:
        return {k: {"s": round(v, 4), "n": self.counts[k]} for k, v in self.seconds.items()}


class Engine:
    def __init__(self, model_dir: str | Path | None = None, settings: EngineSettings | None = None, device: str = "cuda",
                 *, random_config: Mapping[str, Any] | None = None, seed: int = 0):
        """``model_dir``: folder with config.json and safetensors. Or ``random_config`` (a config.json as a dict)
        with ``seed``: random weights drawn on the device."""
        self.settings = s = settings or EngineSettings()
        if (model_dir is None) == (random_config is None):
            raise ValueError("give either a model folder or random_config")
        started = time.perf_counter()
        if model_dir is not None:
            raw, generation = read_config_json(model_dir)
        else:
            raw, generation = dict(random_config), None
        model, self.config = ModelRunner.build_model(raw, generation, dtype=s.dtype, device=device, max_positions=s.max_positions,
                                                      page_size=s.page_size)
        if model_dir is not None:
            load_weights(model, model_dir)
        else:
            fill_random(model, seed)
        self.max_positions = model.runtime.max_positions
        num_pages = s.num_pages
        if num_pages is None:
            per_page = CacheManager.bytes_per_page(model.cache_plan, s.page_size, DTYPES[s.dtype])
            num_pages = max(2, int(s.kv_cache_gb * 2 ** 30 // max(per_page, 1)))
        self.runner = ModelRunner(model, self.config, page_size=s.page_size, num_pages=num_pages, max_requests=s.max_running)
        log.info("cache: %d pages of %d tokens per group; model ready in %.1f s", num_pages, s.page_size,
                 time.perf_counter() - started)
        self.scheduler = Scheduler(self.runner.cache, max_running=s.max_running, max_waiting=s.max_waiting,
                                   max_step_tokens=s.max_step_tokens, prefill_chunk=s.prefill_chunk,
                                   max_positions=self.max_positions, eos_token_ids=model.spec.eos_token_ids,
                                   step_tile=ops.STEP_TILE_ROWS if s.step_tile is None else s.step_tile)
        self.graphs = DecodeGraphs(self.runner, max_batch=s.max_running, max_positions=self.max_positions) if s.cuda_graphs else None
        self._seen: torch.Tensor | None = None  # [slots + 1, vocab] uint8, made when a request first asks for a penalty
        self._done: dict[int, Completion] = {}
        self._callbacks: dict[int, Callable[[Completion], None]] = {}
        self._readback: torch.Tensor | None = None  # pinned: sampled tokens + status word of a step
        self.tokenizer = None
        if model_dir is not None and (Path(model_dir) / "tokenizer.json").is_file():
            from tokenizers import Tokenizer

            self.tokenizer = Tokenizer.from_file(str(Path(model_dir) / "tokenizer.json"))
        self.counters = {"steps": 0, "graph_steps": 0, "prompt_tokens": 0, "generated_tokens": 0, "step_tokens": 0}
        self.profile = StageTimers(s.profile or os.environ.get("OXR_PROFILE") == "1")
        self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if self.profile.enabled else None

    # ---- requests
    def add_request(self, prompt: Sequence[int] | str, params: SamplingParams | None = None,
                    done: Callable[[Completion], None] | None = None) -> Request:
        """Queue a request; raises ``Busy`` when ``max_waiting`` requests are queued already. ``done`` is called with the
        request's ``Completion`` from the ``step()`` in which it ends (oxr_runtime/engine.py:343-371); the returned
        ``Request`` has ``cancel()``."""
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer.json in the model folder; pass token ids instead")
            prompt = self.tokenizer.encode(prompt, add_special_tokens=False).ids
        request = self.scheduler.add([int(t) for t in prompt], params or SamplingParams())
        self.counters["prompt_tokens"] += len(request.prompt_ids)
        if done is not None:
            self._callbacks[request.id] = done
        return request

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    @property
    def preemptions(self) -> int:
        return self.scheduler.preemptions

    # ---- one iteration
    @torch.inference_mode()
    def step(self) -> list[Completion]:
        """Plan one batch, run it, take the sampled tokens; returns the requests that finished."""
        prof = self.profile
        t0 = time.perf_counter() if prof.enabled else 0.0
        plan = self.scheduler.schedule()
        if prof.enabled:
            prof.add("schedule", time.perf_counter() - t0)
            held = sum(r.cache.length for r in self.scheduler.running if r.cache is not None)
        finished = list(plan.finished)
        if plan.entries:
            decode_only = plan.decode_only
            entries = []
            if decode_only:
                # longest context first: the split-KV kernel's blocks start in this order, and a long one that starts
                # last would run on alone (the order stays the same from step to step while the same requests decode)
                plan.entries.sort(key=lambda p: -p.start)
                for p in plan.entries:   # one token each, the last the request holds: hundreds of these per step
                    r = p.request
                    out, params = r.output, r.params
                    entries.append(StepEntry(r.cache, [out[-1] if out else r.prompt_ids[-1]], [0], params.temperature, params.seed,
                                             len(out), params.repetition_penalty))
            else:
                for p in plan.entries:
                    r = p.request
                    entries.append(StepEntry(r.cache, r.tokens_from(p.start, p.count), [p.count - 1] if p.wants_logits else [],
                                             temperature=r.params.temperature, seed=r.params.seed, counter=len(r.output),
                                             penalty=r.params.repetition_penalty))
            try:
                tokens = self._run(plan, entries, decode_only)
            except Exception:
                # every running request fails, the engine stays usable (oxr_runtime/engine.py:483-487,512-516)
                log.exception("step failed")
                finished += self.scheduler.fail_running()
                self._finish(finished)
                raise
            t1 = time.perf_counter() if prof.enabled else 0.0
            wanting = [p.request for p in plan.entries if p.wants_logits]
            finished += self.scheduler.commit(plan, {r.id: t for r, t in zip(wanting, tokens)})
            if prof.enabled:
                prof.add("commit", time.perf_counter() - t1)
                replayed = self._last_step_was_replayed
                device_ms = self._events[0].elapsed_time(self._events[1])
                prof.add("decode_graph" if replayed else "forward", device_ms * 1e-3, plan.tokens)
                prof.steps.append({"ms": device_ms, "tokens": plan.tokens, "graph": replayed, "held": held})
            self.counters["steps"] += 1
            self.counters["step_tokens"] += plan.tokens
            self.counters["generated_tokens"] += len(wanting)
        return self._finish(finished)

    def _finish(self, requests: list[Request]) -> list[Completion]:
        out = []
        for r in requests:
            text = self.tokenizer.decode(r.output, skip_special_tokens=True) if self.tokenizer is not None else None
            c = Scheduler.completion(r, text)
            self._done[r.id] = c
            out.append(c)
            callback = self._callbacks.pop(r.id, None)
            if callback is not None:
                callback(c)
        return out

    def _run(self, plan: StepPlan, entries: list[StepEntry], decode_only: bool) -> list[int]:
        rt = self.runner.model.runtime
        prof = self.profile
        t0 = time.perf_counter() if prof.enabled else 0.0
        if prof.enabled:
            self._events[0].record()
            self._last_step_was_replayed = False
        penalised = any(e.penalty != 1.0 for e in entries)
        if penalised:
            self._mark_new(plan)
        tokens = None
        if self.graphs is not None and decode_only and not penalised:
            replayed = self.graphs.run(entries)
            if replayed is not None:
                # the graph copied the tokens and the status word to pinned memory itself
                self.counters["graph_steps"] += 1
                if prof.enabled:
                    self._events[1].record()
                    self._last_step_was_replayed = True
                    t1 = time.perf_counter()
                    prof.add("build", t1 - t0)
                torch.cuda.current_stream().synchronize()
                if prof.enabled:
                    prof.add("wait", time.perf_counter() - t1)
                host = replayed[1].tolist()
                if host[-2] != 0:
                    ops.check_status(rt.status)
                return host[:len(entries)]
        if tokens is None:
            ctx = self.runner.builder.build(entries)
            logits = self.runner.model.step(ctx, self.runner.cache)
            if logits.shape[0] == 0:
                if prof.enabled:
                    self._events[1].record()
                    prof.add("build", time.perf_counter() - t0)
                    torch.cuda.current_stream().synchronize()
                return []
            s = ctx.sampling
            if penalised:
                ops.repetition_penalty(logits, self._seen, s["row_slot"], s["penalty"])
            sampled = any(e.temperature > 0 for e in entries)
            tokens = ops.sample(logits, s["temperature"], s["seed_lo"], s["seed_hi"], s["counter"]) if sampled else ops.sample(logits)
            if penalised:
                ops.mark_seen(self._seen, s["row_slot"], tokens)
        # one synchronisation per step: the tokens and the kernels' status word land in pinned memory together
        n = tokens.numel()
        if self._readback is None or self._readback.numel() < n + 2:
            self._readback = torch.empty(max(n + 2, 1026), dtype=torch.int32).pin_memory()
        self._readback[:n].copy_(tokens, non_blocking=True)
        self._readback[n:n + 2].copy_(rt.status[:2], non_blocking=True)
        if prof.enabled:
            self._events[1].record()
            t1 = time.perf_counter()
            prof.add("build", t1 - t0)
        torch.cuda.current_stream().synchronize()
        if prof.enabled:
            prof.add("wait", time.perf_counter() - t1)
        host = self._readback[:n + 2].tolist()
        if host[-2] != 0:
            ops.check_status(rt.status)
        return host[:-2]

    def _mark_new(self, plan: StepPlan) -> None:
        """Requests that start (or start again after preemption) with a penalty: mark every token they hold."""
        rt = self.runner.model.runtime
        if self._seen is None:
            self._seen = torch.zeros((self.settings.max_running + 1, self.runner.model.spec.vocab_size), dtype=torch.uint8,
                                     device=rt.device)
        for p in plan.entries:
            r = p.request
            if p.start == 0 and r.params.repetition_penalty != 1.0:
                self._seen[r.cache.state_slot].zero_()
                toks = torch.tensor(r.tokens, dtype=torch.int32, device=rt.device)
                slots = torch.full_like(toks, r.cache.state_slot)
                ops.mark_seen(self._seen, slots, toks)

    # ---- to completion
    def generate(self, prompts: Sequence[Sequence[int] | str], params: SamplingParams | Sequence[SamplingParams] | None = None
                 ) -> list[Completion]:
        """Run the given prompts to completion (blocking); completions come back in the prompts' order."""
        if isinstance(params, SamplingParams) or params is None:
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        requests = []
        pending = list(zip(prompts, params))
        while pending or self.has_work():
            while pending and len(self.scheduler.waiting) < self.scheduler.max_waiting:
                prompt, p = pending.pop(0)
                requests.append(self.add_request(prompt, p))
            self.step()
        return [self._done.pop(r.id) for r in requests]
