"""The Python entry point: ``LLM(model=...).generate(prompt_token_ids, SamplingParams(...))``.

Role in the reference: ``Engine::new`` / ``generate`` / ``begin_request`` / ``step`` / ``poll``
(crates/allpaca-core/src/engine.rs:621, :2895, :3167, :3650, :3661) returning
``GenerationOutput{token_ids, prompt_tokens, completion_tokens, finish_reason}``
(crates/allpaca-types/src/generation.rs:44-50).  The engine works on token ids; text and
tokenizers are outside it.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

from ..config import EngineConfig
from ..sampling import SamplingParams, uniform
from .batch import BatchEntry
from .runner import ModelRunner
from .scheduler import Request, RequestStatus, Scheduler


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str            # "stop" or "length"
    num_preemptions: int = 0

    @property
    def prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def completion_tokens(self) -> int:
        return len(self.token_ids)


class _InFlight:
    """A launched step whose tokens have not been read yet: what was planned, the requests of
    its sampled rows (as planned, and those that were actually run) and the sampler's handle."""

    def __init__(self, out, sampling, live, pending):
        self.out, self.sampling, self.live, self.pending = out, sampling, live, pending


class LLM:
    """One model on one GPU with a continuous-batching scheduler above the step function."""

    def __init__(self, model: Optional[str] = None, dtype="auto", seed: Optional[int] = None,
                 page_size: int = 16, num_pages: Optional[int] = None,
                 max_cache_tokens: Optional[int] = None, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 2048, prefill_chunk: int = 512,
                 max_model_len: Optional[int] = None, gpu_memory_fraction: float = 0.85,
                 device: str = "cuda:0", float32_weights: str = "keep",
                 runner: Optional[ModelRunner] = None, sampler=None):
        """``dtype``: ``"bfloat16"``, ``"float32"`` or ``"auto"`` (what the model folder's
        config.json names as ``torch_dtype``).  ``float32_weights``: what a bfloat16 engine does
        with matrices stored in 32-bit (``"keep"`` and say so, ``"round"``, ``"refuse"``)."""
        if runner is None:
            if model is None:
                raise ValueError("LLM needs a model folder (or a ready runner)")
            cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages,
                               max_cache_tokens=max_cache_tokens, max_num_seqs=max_num_seqs,
                               max_num_batched_tokens=max_num_batched_tokens,
                               prefill_chunk=prefill_chunk, max_model_len=max_model_len,
                               gpu_memory_fraction=gpu_memory_fraction, device=device,
                               float32_weights=float32_weights)
            if seed is not None:
                cfg.seed = seed
            runner = ModelRunner(model, cfg)
        elif seed is not None:
            runner.engine.seed = seed
        self.runner = runner
        e = runner.engine
        self.scheduler = Scheduler(runner.cache, e.max_num_seqs, e.max_num_batched_tokens,
                                   e.prefill_chunk, runner.max_model_len)
        if sampler is None:
            from ..sampling.sampler import Sampler
            sampler = Sampler(runner.device, e.max_num_seqs)
        self.sampler = sampler
        self._ids = itertools.count()
        self._inflight: Optional[_InFlight] = None
        self.stats = {"steps": 0, "prompt_tokens": 0, "tokens_generated": 0, "preemptions": 0,
                      "batched_rows": 0}

    # ---- request-level API ------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int],
                    params: Optional[SamplingParams] = None, request_id: Optional[Hashable] = None) -> Hashable:
        rid = request_id if request_id is not None else next(self._ids)
        req = Request(rid, [int(t) for t in prompt_token_ids], params or SamplingParams())
        vocab = self.runner.vocab_size
        for t in req.prompt_token_ids:
            if not (0 <= t < vocab):
                raise ValueError(f"token {t} out of vocab {vocab}")
        self.scheduler.add(req)
        self.stats["prompt_tokens"] += len(req.prompt_token_ids)
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    def step(self) -> List[RequestOutput]:
        """Launch one batch; returns the requests found finished.

        One step is kept in flight: while the GPU runs the batch launched here, the host reads
        the tokens of the batch before it, appends them and decides who is done.  In steady
        decoding (the same requests, one row each, as in the step before) the new step takes
        its token ids straight from the device, where the step before left them, so the GPU
        never waits for the host.  A request that a stop token ended is therefore known one
        step late: the row it still had in the step in flight is run for nothing and its
        token dropped.  Requests reach the caller one call after the step that finished them;
        :meth:`flush` brings everything up to date."""
        prev = self._inflight
        finished: List[Request] = []
        if prev is not None:
            self.scheduler.advance_counts(prev.out)
            if any(self._at_length_limit(q) for q in prev.live):
                # a request has reached its length limit: it is planned no more, but holds its
                # pages until its last token is here.  Fetch the tokens first, so that the pages
                # are free for the step about to be planned (once per request: no loss).
                finished = self._resolve(prev)
                prev = None
        out = self.scheduler.schedule()
        self.stats["preemptions"] += len(out.preempted)
        if not out.rows:
            if prev is not None:
                finished = finished + self._resolve(prev)
            return self._outputs(finished)
        sampling = [r.request for r in out.rows if r.samples]
        steady = (prev is not None and len(sampling) == len(out.rows) and len(sampling) == len(prev.sampling)
                  and all(r.count == 1 for r in out.rows)
                  and all(a is b for a, b in zip(sampling, prev.sampling)))
        if steady:
            entries = [BatchEntry(r.request.request_id, [0], [0]) for r in out.rows]
            logits = self.runner.step(entries, device_tokens=prev.pending.device)
        else:
            if prev is not None:
                finished = finished + self._resolve(prev)          # the rows planned need the token values
                prev = None
            entries = [BatchEntry(r.request.request_id, r.request.token_slice(r.start, r.count),
                                  [r.count - 1] if r.samples else [])
                       for r in out.rows if r.request.status is not RequestStatus.FINISHED]
            # (a stop token may just have ended a request this step had planned a row for: that
            # row is dropped; the scheduler still counts it among the planned ones)
            logits = self.runner.step(entries) if entries else None
        seed_default = self.runner.engine.seed
        live = [q for q in sampling if q.status is not RequestStatus.FINISHED] if not steady else sampling
        us = [uniform(q.params.seed if q.params.seed is not None else seed_default,
                      len(q.output_token_ids) + q.num_pending) for q in live]
        pending = self.sampler.launch(logits, [q.params for q in live], us) if logits is not None else None
        self.stats["steps"] += 1
        self.stats["batched_rows"] += out.num_tokens
        if steady:
            finished = finished + self._resolve(prev)   # while the GPU runs the step just launched
        self._inflight = _InFlight(out, sampling, live, pending)
        return self._outputs(finished)

    def _at_length_limit(self, q: Request) -> bool:
        n = len(q.output_token_ids) + q.num_pending
        return n >= q.params.max_tokens or len(q.prompt_token_ids) + n >= self.scheduler.max_model_len

    def flush(self) -> List[RequestOutput]:
        """Wait for the step in flight, if any, and record its tokens; returns the requests
        that it finished."""
        prev, self._inflight = self._inflight, None
        if prev is None:
            return []
        self.scheduler.advance_counts(prev.out)
        return self._outputs(self._resolve(prev))

    def _resolve(self, prev: "_InFlight") -> List[Request]:
        """Bring the tokens of a launched step to the host and let the scheduler decide who is
        done.  Rows of requests that had ended before the step ran were not sampled: the
        scheduler is given a filler for them, which it ignores."""
        tokens = self.sampler.fetch(prev.pending) if prev.pending is not None else []
        by_request = {id(q): t for q, t in zip(prev.live, tokens)}
        full = [by_request.get(id(q), 0) for q in prev.sampling]
        finished = self.scheduler.resolve(prev.out, full)
        self.stats["tokens_generated"] += len(tokens)
        if self._inflight is prev:
            self._inflight = None
        for req in finished:
            # a request can end while it holds nothing: preempted (pages given back) while the
            # step with its last row was still in flight, and that row's token was a stop token
            if self.runner.has(req.request_id):
                self.runner.finish(req.request_id)
        return finished

    @staticmethod
    def _outputs(finished: List[Request]) -> List[RequestOutput]:
        return [RequestOutput(req.request_id, req.prompt_token_ids, list(req.output_token_ids),
                              req.finish_reason.value, req.num_preemptions) for req in finished]

    # ---- batch API ----------------------------------------------------------
    def generate(self, prompt_token_ids: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling_params: Union[None, SamplingParams, Sequence[SamplingParams]] = None
                 ) -> List[RequestOutput]:
        """Generate for one prompt or a list of prompts (token ids); outputs in input order."""
        prompts = list(prompt_token_ids)
        if prompts and not isinstance(prompts[0], (list, tuple)):
            prompts = [prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            plist = [sampling_params or SamplingParams()] * len(prompts)
        else:
            plist = list(sampling_params)
            if len(plist) != len(prompts):
                raise ValueError("one SamplingParams per prompt is needed")
        order = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        done: Dict[Hashable, RequestOutput] = {}
        while len(done) < len(order):
            for o in self.step():
                done[o.request_id] = o
        return [done[i] for i in order]
