"""Continuous batching with chunked prefill: which requests run in the next step, with how many tokens each.

One thread, one list of running requests. Each step:

1. every running request that has one token left to compute (a decode) gets that token;
2. what is left of the step's token budget (``max_step_tokens``) goes to running requests still inside their
   prompt, in admission order, each at most ``prefill_chunk`` tokens;
3. then requests are admitted from the head of the waiting queue (never out of order) while a request slot is
   free, budget is left, the cache can take the first portion and, if anything is running, one spare page per
   running request remains (the reference's head-room rule, oxr_runtime/engine.py:433-446).

Logits are wanted only from a request's last token, and only when the portion ends the tokens it has.

When pages run out for a running request, the most recently admitted running request is preempted: its pages
and slot are given back, it keeps the tokens it generated and returns to the FRONT of the waiting queue; when
re-admitted it recomputes prompt + generated tokens and goes on (the reference preempts the same victim but
throws its output away and regenerates, oxr_runtime/engine.py:610-627). If the request that needs the page is
itself the most recent one, it is the one preempted; if it is the only one running, it cannot ever fit and is
finished with ``length`` (oxr_runtime/engine.py:565-569).

The scheduler decides on the host from the cache manager's free lists only; it never touches the device, so its
decisions are tested on the CPU with a stand-in for the model.
"""

from __future__ import annotations

import itertools
import time
from collections import deque
from dataclasses import dataclass, field

from oxr_inference_b200.cache.manager import CacheManager, RequestCache, pages_for
from oxr_inference_b200.sampling.params import Completion, SamplingParams


class Busy(RuntimeError):
    """The waiting queue already holds ``max_waiting`` requests (oxr_runtime/engine.py:139-141,367-368)."""


@dataclass(eq=False)   # a request is itself, not its field values: membership tests and removals compare identities
class Request:
    id: int
    prompt_ids: list[int]
    params: SamplingParams
    output: list[int] = field(default_factory=list)
    cache: RequestCache | None = None
    preemptions: int = 0
    submitted: float = field(default_factory=time.monotonic)
    cancelled: bool = False
    finish_reason: str | None = None
    skipped: int = 0
    """Steps in a row in which the request was running, inside its prompt, and got no tokens."""

    def cancel(self) -> None:
        """Ask for the request to be dropped: at the next step it leaves the queue or gives its pages back and ends with
        ``cancelled`` (oxr_runtime/engine.py:162-171,472-475)."""
        self.cancelled = True

    @property
    def tokens(self) -> list[int]:
        return self.prompt_ids + self.output

    def tokens_from(self, start: int, count: int) -> list[int]:
        """``tokens[start:start + count]`` without joining the two lists first (a decode step asks for one token of each
        of hundreds of long requests)."""
        n = len(self.prompt_ids)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt_ids[start:start + count]
        return self.prompt_ids[start:] + self.output[:start + count - n]

    @property
    def computed(self) -> int:
        return self.cache.length if self.cache is not None else 0

    @property
    def pending(self) -> int:
        """Tokens not yet in the cache; the last of them is the one whose logits give the next token."""
        return len(self.prompt_ids) + len(self.output) - self.computed


@dataclass(slots=True)
class Planned:
    request: Request
    start: int
    count: int
    wants_logits: bool


@dataclass
class StepPlan:
    entries: list[Planned] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    finished: list[Request] = field(default_factory=list)
    """Requests ended while planning (cancelled, or too large for the whole cache)."""

    @property
    def tokens(self) -> int:
        return sum(p.count for p in self.entries)

    @property
    def decode_only(self) -> bool:
        return bool(self.entries) and all(p.count == 1 and p.wants_logits for p in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_running: int, max_waiting: int, max_step_tokens: int,
                 prefill_chunk: int, max_positions: int, eos_token_ids: tuple[int, ...] = (), step_tile: int = 0):
        """``step_tile``: rows of the widest tile of the kernels that will run the step (whoever builds the scheduler asks
        the kernels, or passes a setting); portions are trimmed so that a step's tokens come to whole tile rows. 0: no
        trimming."""
        self.cache = cache
        self.step_tile = int(step_tile)
        self.max_running, self.max_waiting = max_running, max_waiting
        self.max_step_tokens, self.prefill_chunk, self.max_positions = max_step_tokens, prefill_chunk, max_positions
        self.eos = set(eos_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._ids = itertools.count()
        self.preemptions = 0
        """Requests pushed out for lack of pages, cumulative (oxr_runtime/engine.py:268)."""

    # ---- intake
    def add(self, prompt_ids: list[int], params: SamplingParams) -> Request:
        if len(self.waiting) >= self.max_waiting:
            raise Busy(f"{self.max_waiting} requests are already waiting")
        if not prompt_ids:
            raise ValueError("a request needs at least one prompt token")
        if len(prompt_ids) >= self.max_positions:
            raise ValueError(f"a prompt of {len(prompt_ids)} tokens leaves no room under the position limit {self.max_positions}")
        request = Request(next(self._ids), list(prompt_ids), params)
        self.waiting.append(request)
        return request

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step's plan
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        self._drop_cancelled(plan)
        budget = self.max_step_tokens
        chosen: dict[int, Planned] = {}

        def take(request: Request, count: int) -> None:
            nonlocal budget
            chosen[request.id] = Planned(request, request.computed, count, wants_logits=count == request.pending)
            budget -= count

        def make_room(request: Request, count: int) -> bool:
            """``_make_room``; the tokens of requests that it pushed out of this step go back into the budget."""
            nonlocal budget
            before = sum(p.count for p in chosen.values())
            ok = self._make_room(request, count, plan, chosen)
            budget += before - sum(p.count for p in chosen.values())
            return ok

        # 1 and 2: running requests, decodes first, then prompt portions, each group in admission order
        later: list[Request] = []
        for request in list(self.running):
            # a request that was preempted or retired earlier in this pass has no cache any more
            rc = request.cache
            if rc is None:
                continue
            length = rc.length
            if len(request.prompt_ids) + len(request.output) - length != 1:
                later.append(request)
            elif budget > 0 and (length < rc.room or make_room(request, 1)):
                # a single token is never trimmed, and mostly its page is there already
                chosen[request.id] = Planned(request, length, 1, True)
                budget -= 1
        for request in later:
            if request.cache is None:
                continue
            count = self._portion(request, budget)
            if count > 0 and make_room(request, count):
                take(request, count)
                request.skipped = 0
            elif request.cache is not None:
                request.skipped += 1

        # 3: admit from the head of the queue
        while self.waiting and budget > 0 and len(self.running) < self.max_running and self.cache.free_slots > 0:
            request = self.waiting[0]
            count = self._portion(request, budget)
            if count <= 0:
                request.skipped += 1
                break
            needed = pages_for(count, self.cache.page_size)
            if needed > self.cache.usable_pages and not self.running:
                # its first portion alone is beyond the whole cache: shrink the portion to what the cache holds
                count = self.cache.usable_pages * self.cache.page_size
                needed = self.cache.usable_pages
                if count <= 0:
                    break
            if self.running and self.cache.free_pages - needed < len(self.running):
                break
            rc = self.cache.open(request.id)
            if rc is None:
                break
            if not self.cache.reserve(rc, count):
                self.cache.close(rc)
                break
            self.waiting.popleft()
            request.cache = rc
            self.running.append(request)
            take(request, count)
            request.skipped = 0

        plan.entries = [chosen[r.id] for r in self.running if r.id in chosen]
        return plan

    def _portion(self, request: Request, budget: int) -> int:
        """How many of the request's pending tokens this step takes: all of them, or what the chunk size and the step's
        remaining budget allow. With a ``step_tile`` (rows of the widest tile of the kernels: a step of a few tokens more
        than a multiple of it pays for a whole tile row) a portion that does not finish its prompt is trimmed by up to an
        eighth so that the step's tokens so far come to a whole number of tile rows: with tiles of 256 rows, 2,048 prompt
        tokens beside 32 decode tokens would occupy nine tile rows, 2,016 beside 32 occupy eight, and the 32 tokens left
        over ride along with a later step. For the same reason a long step does not take a sliver (less than a tile row)
        of another prompt, unless that prompt got nothing in the step before either: no request waits two steps in a row."""
        count = min(request.pending, self.prefill_chunk, budget)
        planned = self.max_step_tokens - budget
        tile = self.step_tile
        if tile and 0 < count < request.pending:
            if count >= 2 * tile:
                over = (planned + count) % tile
                if 0 < over <= count // 8:
                    count -= over
            elif count < tile and planned >= 2 * tile and (planned + count) % tile and request.skipped == 0:
                count = 0   # a sliver of a prompt at the end of a long step would only open another tile row
        return count

    def _make_room(self, request: Request, count: int, plan: StepPlan, chosen: dict[int, Planned]) -> bool:
        """Reserve pages for ``count`` more tokens of a running request, preempting from the back if needed.
        False if the request itself had to give way (it is then no longer running)."""
        while not self.cache.reserve(request.cache, request.computed + count):
            victim = self.running[-1]
            if victim is request and len(self.running) == 1:
                # alone and still too large: it can never fit
                self._retire(request, "length")
                plan.finished.append(request)
                return False
            self._preempt(victim, plan)
            chosen.pop(victim.id, None)
            if victim is request:
                return False
        return True

    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        self.running.remove(victim)
        self.cache.close(victim.cache)
        victim.cache = None
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)

    def _retire(self, request: Request, reason: str) -> None:
        if request in self.running:
            self.running.remove(request)
        if request.cache is not None:
            self.cache.close(request.cache)
            request.cache = None
        request.finish_reason = reason

    def _drop_cancelled(self, plan: StepPlan) -> None:
        for request in [r for r in self.waiting if r.cancelled]:
            self.waiting.remove(request)
            request.finish_reason = "cancelled"
            plan.finished.append(request)
        for request in [r for r in self.running if r.cancelled]:
            self._retire(request, "cancelled")
            plan.finished.append(request)

    # ---- after the step ran
    def commit(self, plan: StepPlan, sampled: dict[int, int]) -> list[Request]:
        """The step ran: move every planned request forward, take the sampled token of those that wanted one
        (``sampled``: request id -> token) and return the requests that finished."""
        finished = []
        for p in plan.entries:
            request = p.request
            self.cache.advance(request.cache, p.start + p.count)
            if not p.wants_logits:
                continue
            reason = self._take(request, sampled[request.id])
            if reason is not None:
                self._retire(request, reason)
                finished.append(request)
        return finished

    def _take(self, request: Request, token: int) -> str | None:
        """oxr_runtime/engine.py:647-664: an end-of-sequence token ends the request and is not kept."""
        params = request.params
        if (token in self.eos and not params.ignore_eos) or token in params.stop_token_ids:
            return "stop"
        request.output.append(token)
        if len(request.output) >= params.max_tokens:
            return "length"
        if len(request.prompt_ids) + len(request.output) >= self.max_positions:
            return "length"
        return None

    def fail_running(self) -> list[Request]:
        """A step raised: every running request fails, the engine goes on (oxr_runtime/engine.py:512-516)."""
        failed = list(self.running)
        for request in failed:
            self._retire(request, "error")
        return failed

    @staticmethod
    def completion(request: Request, text: str | None = None) -> Completion:
        return Completion(token_ids=list(request.output), finish_reason=request.finish_reason or "unknown",
                          prompt_tokens=len(request.prompt_ids), seconds=time.monotonic() - request.submitted, text=text,
                          preemptions=request.preemptions, request_id=request.id)
