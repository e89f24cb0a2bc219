"""The step function: run one batch of (request, its next tokens) through the model.

``ModelRunner`` owns the model, the cache manager with its device storage, and the
staging buffers.  ``step(entries)`` takes portions of prompts beside single decoded
tokens, cut anywhere, runs only those rows against what earlier steps left in the
cache, and returns 32-bit logits for the rows asked for.  ``finish(request)`` gives a
request's pages and state slot back.  Generation and trace replay both go through it.

Role in the reference: ``forward_batch`` over ``SeqRows``
(crates/allpaca-core/src/model.rs:8839-8885) with page growth by ``ensure_pages``
(model.rs:13452-13480) and release on drop (crates/allpaca-core/src/engine.rs:409-432).
"""
from __future__ import annotations

from typing import Dict, Hashable, Optional, Sequence

import torch

from ..cache import CacheManager, GroupLayout, GroupStorage, StateStorage
from ..config import EngineConfig
from ..models import DecoderModel, load_config
from ..parts import BuildEnv, Workspace
from ..weights import load_checkpoint
from ..ops import library
from .batch import BatchEntry, StepBatch
from .step_builder import build_step


class ModelRunner:
    def __init__(self, model_path: Optional[str], engine: EngineConfig, model: Optional[DecoderModel] = None,
                 model_config=None):
        """Load the model folder at ``model_path`` (or take a ready ``model`` whose weights
        are loaded) and set up caches for it."""
        if engine.dtype in (None, "auto"):
            # the type the checkpoint says it was saved in (config.json's torch_dtype)
            engine.dtype = load_config(model_path)[1].torch_dtype if model_path else "bfloat16"
        engine.validate()
        self.engine = engine
        if not torch.cuda.is_available():
            raise RuntimeError("allpaca_b200 needs a CUDA device (sm_100a); none is visible")
        self.device = torch.device(engine.device)
        torch.cuda.set_device(self.device)
        self.workspace = Workspace(self.device)
        self.env = BuildEnv(dtype=engine.dtype, device=self.device, workspace=self.workspace,
                            page_size=engine.page_size, max_seqs=engine.max_num_seqs)
        if model is None:
            arch, cfg = load_config(model_path)
            model = DecoderModel(arch.spec_builder(cfg), self.env)
            load_checkpoint(model, model_path, engine.dtype, self.device, engine.float32_weights)
            model_config = cfg
        self.model = model
        self.workspace = model.env.workspace      # the buffers the model's parts use
        self.model_config = model_config
        self.vocab_size = model.spec.vocab_size
        self.max_model_len = engine.max_model_len or model.spec.max_position_embeddings
        self._setup_caches()
        self._staging_cap = 0
        self._host = None
        self._dev = None
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}
        # a part that decides on the host what to launch for a step cannot be replayed
        self._host_control = model.host_control()
        self.graph_replays = 0

    # ---- caches ---------------------------------------------------------
    def _setup_caches(self) -> None:
        e = self.engine
        self.cache_plan = self.model.cache_plan()
        page_bytes = [len(g.runs) * g.need.page_bytes(e.page_size, e.dtype) for g in self.cache_plan]
        if e.num_pages is not None:
            num_pages = e.num_pages
        elif e.max_cache_tokens is not None:
            num_pages = -(-e.max_cache_tokens // e.page_size)
        else:
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(free * e.gpu_memory_fraction)
            num_pages = max(1, budget // max(1, sum(page_bytes)))
            # no more than every sequence slot at full length needs
            num_pages = min(num_pages, e.max_num_seqs * -(-self.max_model_len // e.page_size))
        self.num_pages = int(num_pages)
        layouts = [GroupLayout(e.page_size, self.num_pages, g.need.window) for g in self.cache_plan]
        self.cache = CacheManager(layouts, e.max_num_seqs)
        self.storages = [GroupStorage(len(g.runs), self.num_pages, g.need.page_shape(e.page_size),
                                      g.need.dtype or e.dtype, self.device) for g in self.cache_plan]
        self.states = [StateStorage(e.max_num_seqs, b, self.device) if b > 0 else None
                       for b in self.model.state_bytes()]
        self.model.bind_caches(self.cache_plan, self.storages, self.states)

    # ---- requests -------------------------------------------------------
    def has(self, request: Hashable) -> bool:
        return self.cache.has(request)

    def finish(self, request: Hashable) -> None:
        """Give back what the request holds (pages of every group, its state slot)."""
        self.cache.free(request)

    def can_run(self, entries: Sequence[BatchEntry]) -> bool:
        """Whether the pools can supply the pages this batch needs."""
        reserve = [0] * len(self.cache.groups)
        new = 0
        for en in entries:
            req = en.request if self.cache.has(en.request) else None
            if req is None:
                new += 1
            miss = self.cache.pages_missing(req, len(en.tokens))
            for g, m in enumerate(miss):
                reserve[g] += m
        if new > self.engine.max_num_seqs - self.cache.num_running():
            return False
        return all(reserve[g] <= self.cache.num_free_pages(g) for g in range(len(reserve)))

    # ---- the step -------------------------------------------------------
    def step(self, entries: Sequence[BatchEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the rows of ``entries`` as one batch; returns ``[wanted, vocab]`` float32 logits
        in the order of the entries and of their ``want`` lists.  The tensor is a view of a
        buffer that the next step overwrites.

        ``device_tokens`` (int32 on the device, one per row): the step's token ids are taken
        from there instead of from the entries, whose tokens are then placeholders.  With it a
        caller that chooses the next tokens on the GPU can launch the next step without
        bringing them to the host first."""
        if self._graphable(entries):
            logits = self._graph_step(entries, device_tokens)
        else:
            batch = self.prepare(entries, device_tokens=device_tokens)
            logits = self.model.forward(batch)
        if self.cache.has_windows():
            for en in entries:
                self.cache.release_passed(en.request)
        return logits

    # ---- decode steps as CUDA graphs ------------------------------------
    def _graphable(self, entries: Sequence[BatchEntry]) -> bool:
        """A pure decode step (one row per request, every row's logits wanted) of a size
        graphs are kept for."""
        return (self.engine.use_cuda_graphs and not self._host_control
                and 0 < len(entries) <= self.engine.max_num_seqs
                and all(len(en.tokens) == 1 and list(en.want) == [0] for en in entries))

    def _graph_step(self, entries: Sequence[BatchEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Replay (or first capture) the graph of a decode step with ``len(entries)`` rows.

        The graph's kernels read their metadata from buffers at fixed addresses with a
        block-table row as wide as the longest sequence the model takes, so only the
        contents change between replays.  A graph is captured again when a workspace
        buffer it points to has been replaced."""
        B = len(entries)
        # the number of key slices of the attention kernel is part of the graph: graphs are kept
        # per power-of-two bound on the longest context, so it suits the contexts it serves
        held = [self.cache.num_tokens(en.request) if self.cache.has(en.request) else 0 for en in entries]
        longest = max(held) + 1
        bound = 256
        while bound < longest:
            bound *= 2
        bound = min(bound, max(self.max_model_len, 256))
        # ... and per power-of-two bound on the average context, where that lies below the longest:
        # sequences of unequal length want more slices than their number alone suggests
        mean_bound = 256
        while mean_bound < sum(held) // B + 1:
            mean_bound *= 2
        mean_bound = min(mean_bound, bound)
        gs = self._graphs.get((B, bound, mean_bound))
        if gs is None:
            gs = self._graphs[(B, bound, mean_bound)] = _DecodeGraph(self, B)
        batch = self.prepare(entries, staging=gs, widths=gs.widths, device_tokens=device_tokens)
        batch.max_context_len = batch.max_decode_context_len = bound
        batch.mean_context_len = mean_bound
        if gs.graph is not None and gs.generation == self.workspace.generation:
            gs.graph.replay()
            self.graph_replays += 1
            library.add_launches(gs.num_kernels)
            return gs.logits
        # A batch size that shows up once or twice (requests finishing one after another) is
        # run as it is: recording costs about two steps.  From the third use on: run eagerly,
        # which also sizes every buffer, then record.
        gs.uses += 1
        if gs.uses < 3:
            return self.model.forward(batch)
        logits = self.model.forward(batch)
        torch.cuda.current_stream().synchronize()
        before = library.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            gs.logits = self.model.forward(batch)
        gs.num_kernels = library.launch_count() - before
        library.add_launches(-gs.num_kernels)            # recorded, not run
        gs.graph = graph
        gs.generation = self.workspace.generation
        return logits

    def prepare(self, entries: Sequence[BatchEntry], staging=None, widths=None,
                device_tokens: Optional[torch.Tensor] = None) -> StepBatch:
        """Check the batch, allocate its pages and upload its metadata (into ``staging``'s
        fixed buffers with the given block-table widths, when given).

        The checking, the page allocation and the filling of the metadata block are the C++
        step builder's (``csrc/host/step_builder.cpp``); on an error nothing has changed."""
        nseq = len(entries)
        G = len(self.cache.groups)
        T = sum(len(en.tokens) for en in entries)
        R = sum(len(en.want) for en in entries)
        widest = -(-self.max_model_len // min(g.page_size for g in self.cache.groups)) if G else 0
        total_cap = 3 * T + 3 * nseq + 1 + R + nseq * widest * G
        if staging is None:
            host, dev = self._staging(total_cap)
            host_tensor, copied = self._host_tensor, self._copied
        else:
            staging.copied.synchronize()
            host, dev, host_tensor, copied = staging.host, staging.dev, staging.host_tensor, staging.copied
        built = build_step(self.cache, entries, self.vocab_size, self.max_model_len,
                           self.engine.max_num_batched_tokens, host, widths)
        layout, firsts, slots, lens, tok_off = built.layout, built.first_position, built.state_slot, \
            built.query_lens, built.seq_start
        total = int(layout.total)
        dev[:total].copy_(host_tensor[:total], non_blocking=True)
        copied.record()
        if device_tokens is not None:
            if device_tokens.dtype != torch.int32 or device_tokens.numel() < T or not device_tokens.is_cuda:
                raise ValueError("device_tokens must be int32 on the device, one per row of the step")
            dev[layout.off_tokens:layout.off_tokens + T].copy_(device_tokens.reshape(-1)[:T], non_blocking=True)

        def view(off, n):
            return dev[off:off + n]
        tables, off = [], int(layout.off_tables)
        for w in built.table_widths:
            tables.append(view(off, nseq * w).view(nseq, w))
            off += nseq * w
        return StepBatch(
            num_tokens=T, num_seqs=nseq, num_logit_rows=R,
            token_ids=view(layout.off_tokens, T), positions=view(layout.off_positions, T),
            token_seq=view(layout.off_seq, T), seq_start=view(layout.off_start, nseq + 1),
            context_lens=view(layout.off_context, nseq), state_slots=view(layout.off_slot, nseq),
            logit_rows=view(layout.off_rows, R),
            block_tables=tables,
            host_seq_start=tok_off, host_first_position=firsts,
            host_query_lens=lens, host_state_slots=slots,
            max_query_len=int(layout.max_query_len), max_context_len=int(layout.max_context_len),
            **self._decode_contexts(firsts, lens))

    @staticmethod
    def _decode_contexts(firsts, lens) -> dict:
        """Longest and average number of keys of the sequences that bring one row."""
        ones = [f + 1 for f, n in zip(firsts, lens) if n == 1]
        if not ones:
            return {}
        return {"max_decode_context_len": max(ones), "mean_context_len": sum(ones) // len(ones)}

    def _staging(self, n: int):
        if n > self._staging_cap:
            # a step's metadata is read by kernels still in flight: wait before replacing it
            torch.cuda.current_stream().synchronize()
            cap = max(n, 2 * self._staging_cap, 4096)
            self._host_tensor = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._host = self._host_tensor.numpy()
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._staging_cap = cap
            self._copied = torch.cuda.Event()
        else:
            # the previous step's copy out of the pinned buffer must have finished
            self._copied.synchronize()
        return self._host, self._dev

    def memory_report(self) -> Dict[str, int]:
        return {"cache_bytes": sum(s.bytes() for s in self.storages),
                "workspace_bytes": self.workspace.bytes(), "num_pages": self.num_pages}


class _DecodeGraph:
    """Fixed metadata buffers and the captured graph of a decode step with ``B`` rows."""

    def __init__(self, runner: ModelRunner, B: int):
        self.widths = [-(-runner.max_model_len // g.page_size) for g in runner.cache.groups]
        total = 3 * B + (B + 1) + 2 * B + B + sum(B * w for w in self.widths)
        self.host_tensor = torch.empty(total, dtype=torch.int32, pin_memory=True)
        self.host = self.host_tensor.numpy()
        self.dev = torch.empty(total, dtype=torch.int32, device=runner.device)
        self.copied = torch.cuda.Event()
        self.copied.record()
        self.graph = None
        self.logits = None
        self.generation = -1
        self.num_kernels = 0
        self.uses = 0                 # steps of this size so far that found no valid graph
