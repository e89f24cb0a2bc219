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

import torch

from ..config import EngineConfig
from ..sampling import SamplingParams, uniform
from .batch import BatchEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler


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


class LLM:
    """One model on one GPU with a continuous-batching scheduler above the step function."""

    def __init__(self, model: Optional[str] = None, dtype="bfloat16", seed: Optional[int] = None,
                 page_size: int = 16, num_pages: Optional[int] = None,
                 max_cache_tokens: Optional[int] = None, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 2048, prefill_chunk: int = 512,
                 max_model_len: Optional[int] = None, gpu_memory_fraction: float = 0.85,
                 device: str = "cuda:0", runner: Optional[ModelRunner] = None):
        if runner is None:
            if model is None:
                raise ValueError("LLM needs a model folder (or a ready runner)")
            cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages,
                               max_cache_tokens=max_cache_tokens, max_num_seqs=max_num_seqs,
                               max_num_batched_tokens=max_num_batched_tokens,
                               prefill_chunk=prefill_chunk, max_model_len=max_model_len,
                               gpu_memory_fraction=gpu_memory_fraction, device=device)
            if seed is not None:
                cfg.seed = seed
            runner = ModelRunner(model, cfg)
        elif seed is not None:
            runner.engine.seed = seed
        self.runner = runner
        e = runner.engine
        self.scheduler = Scheduler(runner.cache, e.max_num_seqs, e.max_num_batched_tokens,
                                   e.prefill_chunk, runner.max_model_len)
        from ..sampling.sampler import Sampler
        self.sampler = Sampler(runner.device, e.max_num_seqs)
        self._ids = itertools.count()
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
        return self.scheduler.has_unfinished()

    def step(self) -> List[RequestOutput]:
        """Run one batch; returns the requests that finished in it."""
        out = self.scheduler.schedule()
        self.stats["preemptions"] += len(out.preempted)
        if not out.rows:
            return []
        entries = []
        sampling = []
        for r in out.rows:
            toks = r.request.token_slice(r.start, r.count)
            entries.append(BatchEntry(r.request.request_id, toks, [r.count - 1] if r.samples else []))
            if r.samples:
                sampling.append(r.request)
        logits = self.runner.step(entries)
        seed_default = self.runner.engine.seed
        us = [uniform(q.params.seed if q.params.seed is not None else seed_default,
                      len(q.output_token_ids)) for q in sampling]
        tokens = self.sampler.sample(logits, [q.params for q in sampling], us)
        sampled = {q.request_id: t for q, t in zip(sampling, tokens)}
        finished = self.scheduler.advance(out, sampled)
        self.stats["steps"] += 1
        self.stats["batched_rows"] += out.num_tokens
        self.stats["tokens_generated"] += len(tokens)
        outs = []
        for req in finished:
            self.runner.finish(req.request_id)
            outs.append(RequestOutput(req.request_id, req.prompt_token_ids, list(req.output_token_ids),
                                      req.finish_reason.value, req.num_preemptions))
        return outs

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
