"""Decode-only steps replayed from CUDA graphs.

As in the reference (oxr_runtime/decode_graph.py:33-119): batch sizes are rounded up to buckets, the inputs live
in fixed device memory filled from pinned host memory before each replay, rows beyond the real requests point at
a scratch page, and the graph holds the whole step: embedding, every layer, output head and the choice of the
next token. Differences: graphs are captured at first use instead of all at start-up, a graph is keyed by
(batch bucket, block-table width bucket, whether the requests' lengths differ much) so that short contexts do not pay for
the widest possible table and uneven batches get kernels that deal work out by keys rather than by requests, and the
graph also holds the copy of its inputs from pinned memory and the copy of the chosen tokens and the kernels'
status word back to pinned memory: a step is one launch and one synchronisation for the host.
"""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.engine.batch import Layout, StepEntry
from oxr_inference_b200.engine.runtime import ModelRunner
from oxr_inference_b200.parts.base import uneven_lengths

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 192, 256, 384, 512, 768, 1024)  # oxr_runtime/decode_graph.py:30


class DecodeGraphs:
    def __init__(self, runner: ModelRunner, *, max_batch: int, max_positions: int):
        self.runner = runner
        self.buckets = [b for b in BUCKETS if b < max_batch] + [max_batch]
        self.max_width = (max_positions + runner.cache.page_size - 1) // runner.cache.page_size
        self._graphs: dict[tuple[int, int], tuple] = {}
        self._pool = None
        self.kernels_per_replay: dict[tuple[int, int], int] = {}
        self.replays = 0
        self.last_key: tuple[int, int, bool] | None = None
        """(batch bucket, table-width bucket, lengths uneven) of the graph that ``run`` replayed last."""

    def _width_bucket(self, entries: list[StepEntry]) -> int:
        need = max(len(t) for e in entries for t in e.cache.tables)
        w = 16
        while w < need:
            w *= 2
        return min(w, max(self.max_width, need))

    @torch.inference_mode()
    def run(self, entries: list[StepEntry]) -> tuple[torch.Tensor, torch.Tensor] | None:
        """Replay the step for single-token entries. Returns (the chosen tokens on the device, int32, one per entry;
        the pinned host tensor that holds, once the stream has been synchronised, the same tokens followed by the
        first two words of the status word), both overwritten by the next replay; or None when the batch is larger
        than the largest bucket. The caller synchronises before it builds the next step."""
        n = len(entries)
        bucket = next((b for b in self.buckets if b >= n), None)
        if bucket is None:
            return None
        key = (bucket, self._width_bucket(entries), uneven_lengths([e.cache.length + 1 for e in entries]))
        if key not in self._graphs:
            self._capture(key)
        graph, layout, block, tokens, readback = self._graphs[key]
        self.runner.builder.build(entries, layout=layout, device_block=block, copy=False)
        graph.replay()
        self.replays += 1
        self.last_key = key
        ops.launch_count += self.kernels_per_replay[key]
        return tokens[:n], readback

    def _forward(self, ctx) -> torch.Tensor:
        logits = self.runner.model.step(ctx, self.runner.cache)
        s = ctx.sampling
        return ops.sample(logits, s["temperature"], s["seed_lo"], s["seed_hi"], s["counter"])

    @torch.inference_mode()
    def _capture(self, key: tuple[int, int, bool]) -> None:
        bucket, width, uneven = key
        b = self.runner.builder
        m = self.runner.cache
        layout = Layout(bucket, bucket, bucket, [width] * len(m.pools), b.decode_tile_caps(bucket))
        block = torch.zeros(layout.total, dtype=torch.int32, device=b.device)
        # One eager run first, so that whatever is set up at a first call (kernel attributes, plans, workspaces) is set
        # up outside the capture. It runs padding rows only (no entries: every row reads and writes the scratch page and
        # the scratch state slot), so the requests' step runs exactly once, in the replay that follows the capture: a
        # mixer that keeps per-request state must not see a token twice (oxr_runtime/decode_graph.py:84-90 warms up on
        # whatever its static buffers hold, which at start-up is the scratch page as well).
        ctx = b.build([], layout=layout, device_block=block)
        ctx.uneven = uneven      # the fixed block's context keeps it: every replay of this graph has requests of that kind
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward(ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        before = ops.launch_count
        staging = b.staging_of(block)
        readback = torch.zeros(bucket + 2, dtype=torch.int32).pin_memory()
        status = self.runner.model.runtime.status
        # capture_begin / capture_end directly: the `torch.cuda.graph` context also collects garbage and empties the
        # allocator's cache first, which costs a serving engine 0.2 to 0.7 s per new bucket (the capture itself and then
        # every buffer of the next mixed step allocated afresh)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._pool)
            try:
                block.copy_(staging, non_blocking=True)
                tokens = self._forward(ctx)
                readback[:bucket].copy_(tokens, non_blocking=True)
                readback[bucket:].copy_(status[:2], non_blocking=True)
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        self.kernels_per_replay[key] = ops.launch_count - before
        ops.launch_count = before  # capturing launches nothing
        self._graphs[key] = (graph, layout, block, tokens, readback)
