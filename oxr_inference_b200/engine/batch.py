"""Turns a step's host-side description into the device tensors the model reads: one staging block, one copy.

A step is a list of entries (request's cache, its next tokens, which of them want logits). All index arrays the
kernels need (token ids, positions, request boundaries, context lengths, block tables and store slots per cache
group, attention tile lists, rows whose logits are wanted, sampling parameters) are laid out in ONE pinned int32
block and reach the device with ONE asynchronous copy issued before the step's first kernel, as the reference
takes care to do (oxr_runtime/engine.py:523-539, oxr_runtime/decode_graph.py:102-115). With a fixed ``Layout``
(CUDA-graph replay) the device block and every view into it keep their addresses from step to step; rows
beyond the real requests are padding that writes and reads the scratch page (oxr_runtime/decode_graph.py:104-110).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from oxr_inference_b200.cache.manager import CacheManager, RequestCache
from oxr_inference_b200.parts.base import StepContext, uneven_lengths


@dataclass(slots=True)
class StepEntry:
    cache: RequestCache
    tokens: list[int]
    """The request's next tokens, at positions cache.length .. cache.length + len(tokens) - 1."""
    want: list[int]
    """Indices into ``tokens`` whose logits are wanted, in the order wanted."""
    temperature: float = 0.0
    seed: int = 0
    counter: int = 0
    """Index of the output token that will be sampled from this entry's (last) wanted row."""
    penalty: float = 1.0
    """Repetition penalty of the request."""


def _align(n: int) -> int:
    return (n + 3) // 4 * 4


class Layout:
    """Offsets (in int32 words) of every array inside the staging block, for given capacities."""

    def __init__(self, tokens: int, requests: int, rows: int, widths: list[int], tile_caps: dict[tuple[int, int, int], int]):
        self.tokens, self.requests, self.rows, self.widths, self.tile_caps = tokens, requests, rows, list(widths), dict(tile_caps)
        self.offsets: dict[str, tuple[int, int]] = {}
        at = 0

        def put(name: str, size: int) -> None:
            nonlocal at
            self.offsets[name] = (at, size)
            at += _align(max(size, 1))

        for name in ("token_ids", "positions", "req_of_token", "no_store"):
            put(name, tokens)
        put("cu_q", requests + 1)
        put("ctx_lens", requests)
        put("state_slots", requests)
        for name in ("logit_rows", "temperature", "seed_lo", "seed_hi", "counter", "row_slot", "penalty"):
            put(name, rows)
        for g, w in enumerate(widths):
            put(f"slots{g}", tokens)
            put(f"table{g}", requests * w)
        for spec, cap in tile_caps.items():
            put(f"tile_req{spec}", cap)
            put(f"tile_tok0{spec}", cap)
        self.total = at


class BatchBuilder:
    def __init__(self, manager: CacheManager, tile_specs: list[tuple[int, int, int]], device: torch.device, status: torch.Tensor):
        self.manager, self.tile_specs, self.device, self.status = manager, list(tile_specs), device, status
        self._pinned: torch.Tensor | None = None
        self._copied: torch.cuda.Event | None = None
        self._fixed_pinned: dict[int, torch.Tensor] = {}
        self._fixed_views: dict[int, StepContext] = {}
        self._rows: dict[int, list] = {}
        """Per fixed device block: which (request, table version) each block-table row was last filled from, so that
        rows that did not change are not written again."""
        self._same_requests: dict[int, tuple] = {}
        """Per fixed device block: the serials of the requests its rows were last filled for. While the same requests
        decode on, only what moves with a token is written again."""

    # ---- host memory
    def _staging(self, words: int, fixed_block: torch.Tensor | None) -> torch.Tensor:
        """Pinned host memory for one step's arrays. A fixed layout has a staging block of its own, which therefore
        still holds what the layout's previous step wrote."""
        if self._copied is not None:
            self._copied.synchronize()  # the previous step's copy has left its block
            self._copied = None
        if fixed_block is not None:
            key = id(fixed_block)
            if key not in self._fixed_pinned:
                self._fixed_pinned[key] = torch.zeros(words, dtype=torch.int32).pin_memory()
            return self._fixed_pinned[key]
        if self._pinned is None or self._pinned.numel() < words:
            self._pinned = torch.empty(max(words, 4096), dtype=torch.int32).pin_memory()
        return self._pinned

    def staging_of(self, device_block: torch.Tensor) -> torch.Tensor:
        """The pinned block that ``build`` fills for this fixed device block (after its first ``build``)."""
        return self._fixed_pinned[id(device_block)]

    def eager_layout(self, entries: list[StepEntry]) -> Layout:
        m = self.manager
        tokens = sum(len(e.tokens) for e in entries)
        rows = sum(len(e.want) for e in entries)
        widths = [m.table_width([e.cache for e in entries], g) for g in range(len(m.pools))]
        caps = {spec: sum((len(e.tokens) + spec[0] - 1) // spec[0] for e in entries if spec[1] <= len(e.tokens) <= spec[2])
                for spec in self.tile_specs}
        return Layout(tokens, len(entries), rows, widths, caps)

    def decode_tile_caps(self, bucket: int) -> dict[tuple[int, int, int], int]:
        """Single-token requests make one tile each in every list that covers them, none in the others."""
        return {spec: (bucket if spec[1] <= 1 else 0) for spec in self.tile_specs}

    # ---- the build
    @torch.inference_mode()
    def build(self, entries: list[StepEntry], layout: Layout | None = None,
              device_block: torch.Tensor | None = None, copy: bool = True) -> StepContext:
        """Fill the staging block for ``entries`` and copy it. With ``layout``/``device_block`` (graph replay) the
        entries must be single tokens and at most ``layout.requests``; the remaining rows are padding. ``copy=False``
        (fixed layouts only) leaves the copy to the caller, whose graph holds it (``staging_of`` names the source); the
        caller then also sees to it that the step has run before the next ``build`` for this block."""
        m = self.manager
        fixed = layout is not None
        if not fixed:
            layout = self.eager_layout(entries)
        n_real = len(entries)
        if fixed and (n_real > layout.requests or any(len(e.tokens) != 1 or e.want != [0] for e in entries)):
            raise ValueError("a fixed layout takes single-token entries that want their logits, up to its size")
        pinned = self._staging(layout.total, device_block if fixed else None)
        host = pinned.numpy()
        P = m.page_size

        def seg(name: str) -> np.ndarray:
            at, size = layout.offsets[name]
            return host[at:at + size]

        n, T = layout.requests, layout.tokens
        if fixed:
            signature = tuple(e.cache.serial for e in entries)
            known = self._same_requests.get(id(device_block))
            if known is not None and known[0] == signature:
                return self._advance_fixed(entries, layout, device_block, pinned, seg, copy)
        q_lens = [len(e.tokens) for e in entries] + [1] * (n - n_real)
        starts = [e.cache.length for e in entries] + [0] * (n - n_real)
        cu = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu[1:])
        if int(cu[-1]) != T:
            raise ValueError(f"layout holds {T} tokens, the entries bring {int(cu[-1])}")

        ids, pos, req = seg("token_ids"), seg("positions"), seg("req_of_token")
        single = all(q == 1 for q in q_lens)
        if single:   # decode-only step: one assignment per array
            ids[:n_real] = [e.tokens[0] for e in entries]
            ids[n_real:] = 0
            pos[:n_real] = starts[:n_real]
            pos[n_real:] = 0
            req[:] = np.arange(n, dtype=np.int32)
        else:
            ids[:] = 0
            pos[:] = 0
            for i, e in enumerate(entries):
                a, b = int(cu[i]), int(cu[i + 1])
                ids[a:b] = e.tokens
                pos[a:b] = np.arange(starts[i], starts[i] + q_lens[i])
            req[:] = np.repeat(np.arange(n, dtype=np.int32), q_lens)
        seg("no_store")[:] = -1
        seg("cu_q")[:] = cu
        seg("ctx_lens")[:] = [s + q for s, q in zip(starts, q_lens)]
        seg("state_slots")[:] = [e.cache.state_slot for e in entries] + [m.scratch_slot] * (n - n_real)

        rows, temp, slo, shi, cnt, rslot = (seg(k) for k in ("logit_rows", "temperature", "seed_lo", "seed_hi", "counter", "row_slot"))
        temp_f, pen_f = temp.view(np.float32), seg("penalty").view(np.float32)
        if single and all(e.want == [0] for e in entries):
            if layout.rows != n:
                raise ValueError(f"layout holds {layout.rows} logit rows, the entries want {n}")
            rows[:] = np.arange(n, dtype=np.int32)
            temp_f[:n_real] = [e.temperature for e in entries]
            slo[:n_real] = [_as_i32(e.seed & 0xFFFFFFFF) for e in entries]
            shi[:n_real] = [_as_i32((e.seed >> 32) & 0xFFFFFFFF) for e in entries]
            cnt[:n_real] = [e.counter for e in entries]
            rslot[:n_real] = [e.cache.state_slot for e in entries]
            pen_f[:n_real] = [e.penalty for e in entries]
            temp_f[n_real:] = 0.0
            slo[n_real:] = 0
            shi[n_real:] = 0
            cnt[n_real:] = 0
            rslot[n_real:] = m.scratch_slot
            pen_f[n_real:] = 1.0
        else:
            r = 0
            for i, e in enumerate(entries):
                for w in e.want:
                    if not 0 <= w < q_lens[i]:
                        raise ValueError(f"wanted index {w} is outside the entry's {q_lens[i]} tokens")
                    rows[r] = int(cu[i]) + w
                    temp_f[r] = e.temperature
                    slo[r] = _as_i32(e.seed & 0xFFFFFFFF)
                    shi[r] = _as_i32((e.seed >> 32) & 0xFFFFFFFF)
                    cnt[r] = e.counter
                    rslot[r] = e.cache.state_slot
                    pen_f[r] = e.penalty
                    r += 1
            for i in range(n_real, n):  # padding rows: greedy on their own token
                rows[r] = int(cu[i])
                temp_f[r] = 0.0
                slo[r] = shi[r] = cnt[r] = 0
                rslot[r] = m.scratch_slot
                pen_f[r] = 1.0
                r += 1
            if r != layout.rows:
                raise ValueError(f"layout holds {layout.rows} logit rows, the entries want {r}")

        # Block tables: the staging block of a fixed layout keeps last step's rows, so a row whose request and table
        # did not change is left as it is.
        remembered = self._rows.setdefault(id(device_block), [None] * (n * len(m.pools))) if fixed else None
        if remembered is not None and len(remembered) != n * len(m.pools):
            remembered = self._rows[id(device_block)] = [None] * (n * len(m.pools))
        for g in range(len(m.pools)):
            w = layout.widths[g]
            slots, table = seg(f"slots{g}"), seg(f"table{g}").reshape(n, w)
            fill = m.scratch_pages[g] if m.scratch_pages else 0
            for i, e in enumerate(entries):
                key = (e.cache.serial, e.cache.version)   # not id(): a closed request's address is used again
                if remembered is None or remembered[g * n + i] != key:
                    t = e.cache.tables[g]
                    if len(t) > w:
                        raise ValueError(f"a block table of {len(t)} pages does not fit the layout's width {w}")
                    table[i, :len(t)] = t
                    table[i, len(t):] = fill
                    if remembered is not None:
                        remembered[g * n + i] = key
                if q_lens[i] == 1:
                    slots[int(cu[i])] = m.slot(e.cache, g, starts[i])
                else:
                    slots[int(cu[i]):int(cu[i + 1])] = m.slots(e.cache, g, starts[i], starts[i] + q_lens[i])
            for i in range(n_real, n):
                if remembered is None or remembered[g * n + i] != "pad":
                    table[i, :] = fill
                    if remembered is not None:
                        remembered[g * n + i] = "pad"
                slots[int(cu[i])] = fill * P

        tiles_n: dict[tuple[int, int, int], int] = {}
        for spec in self.tile_specs:
            tpt, fewest, most = spec
            treq, ttok = seg(f"tile_req{spec}"), seg(f"tile_tok0{spec}")
            k = 0
            for i, q in enumerate(q_lens):
                if not fewest <= q <= most:
                    continue
                cnt_i = (q + tpt - 1) // tpt
                treq[k:k + cnt_i] = i
                ttok[k:k + cnt_i] = np.arange(cnt_i) * tpt
                k += cnt_i
            tiles_n[spec] = k

        if device_block is None:
            device_block = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        if copy or not fixed:
            device_block[:layout.total].copy_(pinned[:layout.total], non_blocking=True)
            self._copied = torch.cuda.Event()
            self._copied.record()
        ctx_lens = [s + q for s, q in zip(starts, q_lens)]
        if fixed:   # the views into a fixed block never change: make them once
            self._same_requests[id(device_block)] = (signature,)
            ctx = self._fixed_views.get(id(device_block))
            if ctx is None:
                ctx = self._fixed_views[id(device_block)] = self.views(layout, device_block, tiles_n, q_lens, ctx_lens, max(layout.widths) * P)
            ctx.q_lens, ctx.ctx_lens_host = q_lens, ctx_lens
            return ctx
        ctx = self.views(layout, device_block, tiles_n, q_lens, ctx_lens, max(ctx_lens))
        ctx.uneven = uneven_lengths(ctx_lens)
        return ctx

    def _advance_fixed(self, entries: list[StepEntry], layout: Layout, device_block: torch.Tensor, pinned: torch.Tensor, seg,
                       copy: bool) -> StepContext:
        """The same requests as in this block's last step, each one token further: the staging block still holds
        everything that belongs to a request as such (its rows, sampling parameters, state slot, tile entries, the
        padding); written again are the token, its position and cache slot, the context length, the output index
        and a block-table row whose request got or gave back a page."""
        m = self.manager
        n, n_real = layout.requests, len(entries)
        starts = [e.cache.length for e in entries]
        seg("token_ids")[:n_real] = [e.tokens[0] for e in entries]
        seg("positions")[:n_real] = starts
        seg("ctx_lens")[:n_real] = [s + 1 for s in starts]
        seg("counter")[:n_real] = [e.counter for e in entries]
        remembered = self._rows[id(device_block)]
        P = m.page_size
        for g in range(len(m.pools)):
            w = layout.widths[g]
            table = None
            slots = []
            for i, e in enumerate(entries):
                rc = e.cache
                key = (rc.serial, rc.version)
                t = rc.tables[g]
                if remembered[g * n + i] != key:
                    if table is None:
                        table = seg(f"table{g}").reshape(n, w)
                    if len(t) > w:
                        raise ValueError(f"a block table of {len(t)} pages does not fit the layout's width {w}")
                    table[i, :len(t)] = t
                    table[i, len(t):] = m.scratch_pages[g] if m.scratch_pages else 0
                    remembered[g * n + i] = key
                page = t[starts[i] // P]
                if page < 0:
                    raise ValueError("a position to be written lies on a released page")
                slots.append(page * P + starts[i] % P)
            seg(f"slots{g}")[:n_real] = slots   # one write for all requests: hundreds of them per step
        if copy:
            device_block[:layout.total].copy_(pinned[:layout.total], non_blocking=True)
            self._copied = torch.cuda.Event()
            self._copied.record()
        ctx = self._fixed_views[id(device_block)]
        ctx.q_lens, ctx.ctx_lens_host = [1] * n, [s + 1 for s in starts] + [1] * (n - n_real)
        return ctx

    def views(self, layout: Layout, block: torch.Tensor, tiles_n: dict, q_lens: list[int], ctx_lens: list[int],
              kv_len_bound: int) -> StepContext:
        m = self.manager

        def dev(name: str) -> torch.Tensor:
            at, size = layout.offsets[name]
            return block[at:at + size]

        groups = [m.group_view(g, dev(f"table{g}").view(layout.requests, layout.widths[g]), dev(f"slots{g}"))
                  for g in range(len(m.pools))]
        ctx = StepContext(
            n_tokens=layout.tokens, n_requests=layout.requests, token_ids=dev("token_ids"), positions=dev("positions"),
            req_of_token=dev("req_of_token"), cu_q=dev("cu_q"), ctx_lens=dev("ctx_lens"), state_slots=dev("state_slots"),
            logit_rows=dev("logit_rows"), no_store_slots=dev("no_store"), groups=groups,
            tiles={t: (dev(f"tile_req{t}"), dev(f"tile_tok0{t}"), tiles_n[t]) for t in self.tile_specs},
            kv_len_bound=kv_len_bound, q_lens=q_lens, ctx_lens_host=ctx_lens, status=self.status,
        )
        ctx.sampling = {"temperature": dev("temperature").view(torch.float32), "seed_lo": dev("seed_lo"),
                        "seed_hi": dev("seed_hi"), "counter": dev("counter"), "row_slot": dev("row_slot"),
                        "penalty": dev("penalty").view(torch.float32)}
        return ctx


def _as_i32(u: int) -> int:
    """Reinterpret an unsigned 32-bit value as the int32 with the same bits."""
    return u - (1 << 32) if u >= (1 << 31) else u
