"""Continuous batching: which requests run which tokens in the next step.

The decisions are made by the C++ scheduler (``csrc/host/scheduler.cpp``, part of the host
library that also holds the cache manager and the step builder); this module keeps the
requests' token lists and sampling parameters, which native code never needs, and mirrors
the few fields callers read (status, tokens computed, preemptions).

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
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import ctypes

from ..cache import CacheManager
from ..cache.manager import host_library
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
    num_pending: int = 0                  # tokens sampled on the device whose values are not here yet

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
    """The Python face of the native scheduler."""

    _REASONS = {1: FinishReason.STOP, 2: FinishReason.LENGTH}

    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk: int, max_model_len: int):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.token_budget = max_num_batched_tokens
        self.prefill_chunk = prefill_chunk
        self.max_model_len = max_model_len
        self._lib = host_library()
        self._h = self._lib.aps_create(cache.native, int(max_num_seqs), int(max_num_batched_tokens),
                                       int(prefill_chunk), int(max_model_len))
        if not self._h:
            raise ValueError("the scheduler needs a positive number of sequences, token budget, portion "
                             "size and length limit")
        self._requests: Dict[int, Request] = {}          # number -> request, while running or waiting
        self._arrivals = 0
        self._counts = (ctypes.c_int * 3)()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.aps_destroy(self._h)
            self._h = None

    def _error(self) -> str:
        return self._lib.apc_last_error().decode()

    # ---- adding ---------------------------------------------------------
    def add(self, request: Request) -> None:
        known = request.request_id in self.cache._pinned
        n = self.cache.pin(request.request_id)
        stops = request.params.stop_token_ids
        arr = (ctypes.c_int * max(len(stops), 1))(*stops)
        rc = self._lib.aps_add(self._h, n, len(request.prompt_token_ids), int(request.params.max_tokens),
                               arr, len(stops))
        if rc != 0:
            if not known:
                self.cache.unpin(request.request_id)
            raise AdmissionError(f"request {request.request_id!r}: {self._error()}")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.status = RequestStatus.WAITING
        self._requests[n] = request

    def adopt_running(self, request: Request, num_computed: int) -> None:
        """A request whose first ``num_computed`` prompt tokens are already in the cache (put
        there by the caller) joins the running requests."""
        n = self.cache.pin(request.request_id)
        rc = self._lib.aps_adopt_running(self._h, n, len(request.prompt_token_ids),
                                         int(request.params.max_tokens), int(num_computed))
        if rc != 0:
            self.cache.unpin(request.request_id)
            raise AdmissionError(f"request {request.request_id!r}: {self._error()}")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.num_computed = int(num_computed)
        request.status = RequestStatus.RUNNING
        self._requests[n] = request

    def has_unfinished(self) -> bool:
        return bool(self._lib.aps_has_unfinished(self._h))

    def _listed(self, which: int) -> List[Request]:
        cap = max(len(self._requests), 1)
        buf = (ctypes.c_int64 * cap)()
        n = self._lib.aps_list(self._h, which, buf, cap)
        return [self._requests[buf[i]] for i in range(min(n, cap))]

    @property
    def running(self) -> List[Request]:
        """The running requests in the scheduler's order (a copy)."""
        return self._listed(0)

    @property
    def waiting(self) -> List[Request]:
        """The waiting requests, the next to be admitted first (a copy)."""
        return self._listed(1)

    # ---- one step -------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        rc = self._lib.aps_schedule(self._h, self._counts)
        if rc != 0:
            raise RuntimeError(self._error())
        nrows, npre, nadm = self._counts[0], self._counts[1], self._counts[2]
        rows_buf = (ctypes.c_int64 * max(4 * nrows, 1))()
        pre_buf = (ctypes.c_int64 * max(npre, 1))()
        adm_buf = (ctypes.c_int64 * max(nadm, 1))()
        self._lib.aps_planned(self._h, rows_buf, pre_buf, adm_buf)
        reqs = self._requests
        preempted = []
        for i in range(npre):
            req = reqs[pre_buf[i]]
            req.num_computed = 0
            req.status = RequestStatus.WAITING
            req.num_preemptions += 1
            self.cache.forget(req.request_id)        # native code has freed its pages and slot
            preempted.append(req)
        for i in range(nadm):
            reqs[adm_buf[i]].status = RequestStatus.RUNNING
        rows = [ScheduledRows(reqs[rows_buf[4 * i]], rows_buf[4 * i + 1], rows_buf[4 * i + 2],
                              bool(rows_buf[4 * i + 3])) for i in range(nrows)]
        return SchedulerOutput(rows, preempted)

    # ---- after the step -------------------------------------------------
    def advance(self, output: SchedulerOutput, sampled: Dict[Hashable, int]) -> List[Request]:
        """Record the step: rows are now cached; sampled tokens are appended; requests that
        are done are taken out (their cache is the caller's to free).  Returns them."""
        self.advance_counts(output)
        return self.resolve(output, [int(sampled[r.request.request_id]) for r in output.rows if r.samples])

    def advance_counts(self, output: SchedulerOutput) -> None:
        """First half of :meth:`advance`, for a caller that launches the next step before this
        step's tokens have reached the host: the step has been launched, its rows count as
        cached and every sampled row's request as one token longer (value still unknown)."""
        rc = self._lib.aps_advance_counts(self._h)
        if rc != 0:
            raise RuntimeError(self._error())
        for r in output.rows:
            if r.request.status is not RequestStatus.FINISHED:
                r.request.num_computed += r.count
                if r.samples:
                    r.request.num_pending += 1

    def resolve(self, output: SchedulerOutput, tokens: Sequence[int]) -> List[Request]:
        """Second half: the token values of the oldest step not yet resolved, one per sampled
        row in order.  Appends them (except to requests a stop token ended a step earlier),
        decides who is done and returns those; their cache is the caller's to free."""
        toks = [int(t) for t in tokens]
        arr = (ctypes.c_int * max(len(toks), 1))(*toks)
        nfin = ctypes.c_int(0)
        rc = self._lib.aps_resolve(self._h, arr, len(toks), ctypes.byref(nfin))
        if rc != 0:
            raise RuntimeError(self._error())
        k = 0
        for r in output.rows:
            if not r.samples:
                continue
            if r.request.status is not RequestStatus.FINISHED:
                r.request.output_token_ids.append(toks[k])
                r.request.num_pending -= 1
            k += 1
        finished: List[Request] = []
        if nfin.value:
            ids = (ctypes.c_int64 * nfin.value)()
            reasons = (ctypes.c_int * nfin.value)()
            self._lib.aps_finished(self._h, ids, reasons)
            for i in range(nfin.value):
                req = self._requests.pop(ids[i])
                req.finish_reason = self._REASONS[reasons[i]]
                req.status = RequestStatus.FINISHED
                self.cache.unpin(req.request_id)
                finished.append(req)
        return finished

    def unresolved_steps(self) -> int:
        return int(self._lib.aps_unresolved_steps(self._h))

    def abort(self, request_id: Hashable) -> Optional[Request]:
        """Take a request out, running or waiting; its cache is the caller's to free."""
        n = self.cache._numbers.get(request_id)
        if n is None or n not in self._requests:
            return None
        self._lib.aps_abort(self._h, n)
        req = self._requests.pop(n)
        req.status = RequestStatus.FINISHED
        self.cache.unpin(request_id)
        return req
