"""One step's batch: rows of several requests, flattened, with the metadata kernels read.

A batch holds, per request, the next tokens to run: a portion of a prompt (any length, cut
anywhere) or a single decoded token.  Rows of a request are contiguous and in order.

Role in the reference: ``SeqRows{start_pos, n_rows, page_ids, request_id}`` and the
concatenated token list of ``forward_batch`` (crates/allpaca-core/src/model.rs:36-42,
:8839-8848, :10865-10885).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Sequence

import torch


@dataclass
class BatchEntry:
    """The rows one request contributes to a step."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()        # indices into `tokens` whose logits are asked for


@dataclass
class StepBatch:
    """Device tensors and host facts of one step (built by :class:`BatchBuilder`)."""

    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    token_ids: torch.Tensor            # [T] int32
    positions: torch.Tensor            # [T] int32, absolute position of each row
    token_seq: torch.Tensor            # [T] int32, index of the row's request in this batch
    seq_start: torch.Tensor            # [nseq+1] int32, first row of each request
    context_lens: torch.Tensor         # [nseq] int32, tokens held after this step
    state_slots: torch.Tensor          # [nseq] int32
    logit_rows: torch.Tensor           # [R] int32 rows whose logits are returned
    block_tables: List[torch.Tensor]   # per cache group: [nseq, max_pages] int32
    # host copies for parts that walk sequences themselves
    host_seq_start: List[int] = field(default_factory=list)
    host_query_lens: List[int] = field(default_factory=list)
    host_first_position: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    shared: dict = field(default_factory=dict)    # per-step values parts share (cleared per forward)
    max_query_len: int = 0
    max_context_len: int = 0
    # of the sequences that bring one row, whose attention is cut into key slices by these two
    # (0: not known; the longest context of all stands in)
    max_decode_context_len: int = 0
    mean_context_len: int = 0
