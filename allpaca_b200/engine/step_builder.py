"""One step's batch, built on the host by the C++ step builder.

``build_step`` hands a step's rows to ``csrc/host/step_builder.cpp``, which checks them
(tokens inside the vocabulary, wanted rows inside the portion, length limits, no request
twice), makes room for them in the cache manager and fills the block of 32-bit integers the
kernels read.  Nothing here touches a GPU.  On an error nothing has changed.

Role in the reference: the concatenated token list and ``SeqRows`` of ``forward_batch``
(crates/allpaca-core/src/model.rs:36-42, :8839-8848), the token check (:8215-8219) and page
growth by ``ensure_pages`` (:13452-13480).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from ..cache.manager import CacheManager, OutOfPages, host_library
from .batch import BatchEntry


class StepError(ValueError):
    """A batch the step function cannot run (caller's mistake); nothing was changed."""


class StepLayout(ctypes.Structure):
    """Where the step builder put each array of the metadata block (``ApcStepLayout``)."""

    _fields_ = [("num_tokens", ctypes.c_int32), ("num_seqs", ctypes.c_int32), ("num_logit_rows", ctypes.c_int32),
                ("max_query_len", ctypes.c_int32), ("max_context_len", ctypes.c_int32), ("pad", ctypes.c_int32),
                ("total", ctypes.c_int64), ("off_tokens", ctypes.c_int64), ("off_positions", ctypes.c_int64),
                ("off_seq", ctypes.c_int64), ("off_start", ctypes.c_int64), ("off_context", ctypes.c_int64),
                ("off_slot", ctypes.c_int64), ("off_rows", ctypes.c_int64), ("off_tables", ctypes.c_int64)]


@dataclass
class BuiltStep:
    layout: StepLayout
    table_widths: List[int]        # per cache group; the tables lie one after another from off_tables
    first_position: List[int]      # position of each request's first row
    state_slot: List[int]
    query_lens: List[int]
    seq_start: List[int]           # first row of each request, and the total


def build_step(cache: CacheManager, entries: Sequence[BatchEntry], vocab_size: int, max_model_len: int,
               max_batched_tokens: int, host: np.ndarray, fixed_widths: Optional[Sequence[int]] = None
               ) -> BuiltStep:
    """Fill ``host`` (int32) with the step's metadata; see :class:`StepLayout` for the places."""
    if not entries:
        raise StepError("a step needs at least one entry")
    nseq = len(entries)
    lens = np.fromiter((len(en.tokens) for en in entries), dtype=np.int32, count=nseq)
    wlens = np.fromiter((len(en.want) for en in entries), dtype=np.int32, count=nseq)
    tok_off = np.zeros(nseq + 1, dtype=np.int32)
    np.cumsum(lens, out=tok_off[1:])
    want_off = np.zeros(nseq + 1, dtype=np.int32)
    np.cumsum(wlens, out=want_off[1:])
    T, R = int(tok_off[-1]), int(want_off[-1])
    try:
        tokens = np.fromiter((t for en in entries for t in en.tokens), dtype=np.int64, count=T)
        want = np.fromiter((w for en in entries for w in en.want), dtype=np.int64, count=R)
    except (TypeError, ValueError) as e:
        raise StepError(f"token ids and wanted rows must be integers: {e}") from None
    for arr, what in ((tokens, "token"), (want, "wanted row")):
        if arr.size and (arr.min() < -2 ** 31 or arr.max() >= 2 ** 31):
            raise StepError(f"{what} {int(arr.max())} is out of range")
    tokens, want = tokens.astype(np.int32), want.astype(np.int32)
    if len({en.request for en in entries}) != nseq:
        raise StepError("a request appears twice in one step")
    # new requests get their handles now; they are dropped again if the step is refused
    fresh = [en.request for en in entries if not cache.has(en.request)]
    reqs = np.fromiter((cache.handle(en.request) if cache.has(en.request) else cache.adopt(en.request)
                        for en in entries), dtype=np.int64, count=nseq)
    fixed = np.asarray(fixed_widths, dtype=np.int32) if fixed_widths is not None else None
    layout = StepLayout()
    firsts = np.zeros(nseq, dtype=np.int64)
    slots = np.zeros(nseq, dtype=np.int32)
    widths = np.zeros(max(1, len(cache.groups)), dtype=np.int32)
    lib = host_library()
    rc = lib.apc_prepare_step(
        cache.native, int(vocab_size), int(max_model_len), int(max_batched_tokens), nseq,
        reqs.ctypes.data, tok_off.ctypes.data, tokens.ctypes.data, want_off.ctypes.data, want.ctypes.data,
        fixed.ctypes.data if fixed is not None else None, host.ctypes.data, host.shape[0],
        ctypes.addressof(layout), widths.ctypes.data, firsts.ctypes.data, slots.ctypes.data)
    if rc != 0:
        for r in fresh:
            cache.forget(r)
        msg = lib.apc_last_error().decode()
        if rc == 2:
            raise OutOfPages(msg)
        raise StepError(msg)
    return BuiltStep(layout, widths[:len(cache.groups)].tolist(), firsts.tolist(), slots.tolist(), lens.tolist(),
                     tok_off.tolist())
