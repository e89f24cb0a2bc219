"""Continuous batching: which requests run which tokens in the next step.

Every step is one batch under a token budget: first one row for each running request
that is decoding, then portions of running prompts, then newly admitted requests, in
order of arrival.  A prompt is cut into portions of at most ``prefill_chunk`` tokens
and whatever the budget leaves.  A request's last scheduled row yields logits (and a
sampled token) only when the step completes everything the request holds so far.

When pages run out: a row that cannot get its page makes the scheduler preempt the
running request that arrived last (possibly the one asking): its pages and state slot
are given back, and it returns to the head of the waiting queue to be recomputed later
with the tokens it has already produced kept as part of its prompt.  A prompt portion
that does not fit is shortened to the pages that are free, or waits.  A request that
could never fit in an empty pool is refused when it is added, so one request can
always run to its end and the queue cannot starve.

Role in the reference: admission in ``begin_request`` with a hard cap and no queue
(crates/allpaca-core/src/engine.rs:3198), one prefill chunk per tick (:4717, :4756), the
fair pick of ``pick_runnable`` (crates/allpaca-core/src/scheduler.rs:647-664), batched decode
of all plain decoders (engine.rs:5451-5560) and finish reasons (:4607-4621).  The reference
never mixes a prompt chunk with decode rows (engine.rs:5430) and never preempts (it spills
pages to slower tiers, crates/allpaca-core/src/kv_tier.rs:1939-1961); both are design choices
of this engine.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional

from ..cache import CacheManager
from ..sampling.params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(enum.Enum):
    STOP = "stop"        # a stop token was produced (it is part of the output ids)
    LENGTH = "length"    # max_tokens new tokens, or the model's length limit


class AdmissionError(ValueError):
    """A request this engine can never run."""


@dataclass
class Request:
    request_id: Hashable
    prompt_token_ids: List[int]
    params: SamplingParams
    arrival: int = 0
    output_token_ids: List[int] = field(default_factory=list)
    num_computed: int = 0                 # tokens whose keys and values are in the cache
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: Optional[FinishReason] = None
    num_preemptions: int = 0

    @property
    def all_token_ids(self) -> List[int]:
        return self.prompt_token_ids + self.output_token_ids

    def token_slice(self, start: int, count: int) -> List[int]:
        """``all_token_ids[start:start + count]`` without joining the two lists (a decode step
        asks for one token of a sequence that may be very long)."""
        n = len(self.prompt_token_ids)
        end = start + count
        if end <= n:
            return self.prompt_token_ids[start:end]
        if start >= n:
            return self.output_token_ids[start - n:end - n]
        return self.prompt_token_ids[start:] + self.output_token_ids[:end - n]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)


@dataclass
class ScheduledRows:
    request: Request
    start: int           # index of the first scheduled token in all_token_ids
    count: int
    samples: bool        # the last row completes the request's tokens: sample from it


@dataclass
class SchedulerOutput:
    rows: List[ScheduledRows]
    preempted: List[Request]

    @property
    def num_tokens(self) -> int:
        return sum(r.count for r in self.rows)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk: int, max_model_len: int):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.token_budget = max_num_batched_tokens
        self.prefill_chunk = prefill_chunk
        self.max_model_len = max_model_len
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0

    # ---- adding ---------------------------------------------------------
    def add(self, request: Request) -> None:
        n = len(request.prompt_token_ids)
        if n == 0:
            raise AdmissionError("a request needs at least one prompt token")
        if n >= self.max_model_len:
            raise AdmissionError(f"a prompt of {n} tokens leaves no room under the model's "
                                 f"length limit {self.max_model_len}")
        longest = min(n + request.params.max_tokens, self.max_model_len)
        for g, layout in enumerate(self.cache.groups):
            need = -(-longest // layout.page_size)
            if layout.window is not None:
                # a windowed group keeps at most the window plus one step's rows alive
                span = layout.window + min(self.prefill_chunk, self.token_budget) + layout.page_size
                need = min(need, -(-span // layout.page_size) + 1)
            if need > layout.num_pages:
                raise AdmissionError(
                    f"request {request.request_id!r} may hold {longest} tokens = {need} pages of "
                    f"cache group {g}, whose pool has {layout.num_pages}")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.status = RequestStatus.WAITING
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step -------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        budget = self.token_budget
        rows: List[ScheduledRows] = []
        preempted: List[Request] = []
        reserved = [0] * len(self.cache.groups)

        def fits(req: Request, count: int) -> bool:
            key = req.request_id if self.cache.has(req.request_id) else None
            return self.cache.can_append(key, count, reserved)

        def reserve(req: Request, count: int) -> None:
            key = req.request_id if self.cache.has(req.request_id) else None
            for g, m in enumerate(self.cache.pages_missing(key, count)):
                reserved[g] += m

        # 1. decode rows of running requests, oldest first; preempt the youngest on shortage
        self.running.sort(key=lambda r: r.arrival)
        decoding = [r for r in self.running if r.num_tokens - r.num_computed == 1]
        i = 0
        while i < len(decoding):
            req = decoding[i]
            if budget <= 0:
                break
            if fits(req, 1):
                reserve(req, 1)
                rows.append(ScheduledRows(req, req.num_computed, 1, True))
                budget -= 1
                i += 1
                continue
            victim = max(self.running, key=lambda r: r.arrival)
            self._preempt(victim)
            preempted.append(victim)
            # drop rows already planned for the victim and what they had reserved
            if any(r.request is victim for r in rows):
                rows = [r for r in rows if r.request is not victim]
                budget = self.token_budget - sum(r.count for r in rows)
                reserved = [0] * len(self.cache.groups)
                for r in rows:
                    reserve(r.request, r.count)
            decoding = [r for r in decoding if r is not victim]
            if victim is req:
                continue

        # 2. portions of running prompts; if every running request is starved of pages,
        #    preempt the youngest and try again
        while True:
            for req in self.running:
                if budget <= 0:
                    break
                left = req.num_tokens - req.num_computed
                if left <= 1:
                    continue
                count = self._largest_fit(req, min(left, budget, self.prefill_chunk), reserved)
                if count <= 0:
                    continue
                reserve(req, count)
                rows.append(ScheduledRows(req, req.num_computed, count, count == left))
                budget -= count
            if rows or not self.running:
                break
            victim = max(self.running, key=lambda r: r.arrival)
            self._preempt(victim)
            preempted.append(victim)

        # 3. admit waiting requests in order while all the tokens they hold would fit;
        #    stop at the first that does not
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs \
                and self.cache.can_begin():
            req = self.waiting[0]
            left = req.num_tokens - req.num_computed
            if not self.cache.can_append(None, left, reserved):
                break
            count = min(left, budget, self.prefill_chunk)
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            reserve(req, count)
            rows.append(ScheduledRows(req, req.num_computed, count, count == left))
            budget -= count

        if not rows and self.has_unfinished() and not preempted:
            raise RuntimeError("the scheduler found nothing to run although requests are pending")
        return SchedulerOutput(rows, preempted)

    def _largest_fit(self, req: Request, want: int, reserved) -> int:
        """The most tokens up to ``want`` whose pages are free (0 if not even one)."""
        key = req.request_id if self.cache.has(req.request_id) else None
        if want <= 0:
            return 0
        if self.cache.can_append(key, want, reserved):
            return want
        lo, hi = 0, want                     # can_append(lo) holds or lo == 0
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.cache.can_append(key, mid, reserved):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        if self.cache.has(req.request_id):
            self.cache.free(req.request_id)
        req.num_computed = 0
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.waiting.appendleft(req)

    # ---- after the step -------------------------------------------------
    def advance(self, output: SchedulerOutput, sampled: Dict[Hashable, int]) -> List[Request]:
        """Record the step: rows are now cached; sampled tokens are appended; requests that
        are done are taken out (their cache is the caller's to free).  Returns them."""
        finished: List[Request] = []
        for r in output.rows:
            req = r.request
            req.num_computed += r.count
            if not r.samples:
                continue
            tok = sampled[req.request_id]
            req.output_token_ids.append(int(tok))
            reason = self._finish_reason(req, int(tok))
            if reason is not None:
                req.finish_reason = reason
                req.status = RequestStatus.FINISHED
                self.running.remove(req)
                finished.append(req)
        return finished

    def _finish_reason(self, req: Request, tok: int) -> Optional[FinishReason]:
        # stop wins over length (crates/allpaca-core/src/engine.rs:4607-4621)
        if tok in req.params.stop_token_ids:
            return FinishReason.STOP
        if len(req.output_token_ids) >= req.params.max_tokens:
            return FinishReason.LENGTH
        if req.num_tokens >= self.max_model_len:
            return FinishReason.LENGTH
        return None

    def abort(self, request_id: Hashable) -> Optional[Request]:
        for req in list(self.running):
            if req.request_id == request_id:
                self.running.remove(req)
                req.status = RequestStatus.FINISHED
                return req
        for req in list(self.waiting):
            if req.request_id == request_id:
                self.waiting.remove(req)
                req.status = RequestStatus.FINISHED
                return req
        return None
