"""Trace replay: drive the step function with given tokens and dump logits.

It owns no forward pass, cache or loader: it builds the same :class:`ModelRunner` that
generation uses and calls its ``step`` and ``finish``.

Role in the reference: the logits taps ``Engine::tap_logits`` / ``ALLPACA_LOGITS_DUMP``
(crates/allpaca-core/src/engine.rs:1179-1188, crates/allpaca-core/src/sampling.rs:104-127)
and the per-row logits of ``forward_tokens`` (crates/allpaca-core/src/model.rs:8889-8890);
the reference has no stand-alone replay program.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence

PAGE_SIZE = 16      # divides 64, the rounding unit of --max-tokens
MAX_LIVE = 4


def parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--page-size", type=int, default=PAGE_SIZE)
    p.add_argument("--max-live", type=int, default=MAX_LIVE, help="requests live at a time")
    p.add_argument("--no-graphs", action="store_true",
                   help="launch every kernel from the host (as generation does, steps of one row per request "
                        "are otherwise replayed as CUDA graphs from their third use on)")
    return p.parse_args(argv)


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = parse_args(argv)
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    import torch
    from ..config import EngineConfig
    from .batch import BatchEntry
    from .runner import ModelRunner

    if 64 % args.page_size != 0:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 2
    rounded = -(-args.max_tokens // 64) * 64
    cfg = EngineConfig(dtype=args.dtype, page_size=args.page_size,
                       num_pages=rounded // args.page_size, max_num_seqs=args.max_live,
                       max_num_batched_tokens=max(rounded, args.max_live), prefill_chunk=rounded,
                       use_cuda_graphs=not args.no_graphs)
    runner = ModelRunner(args.model, cfg)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [BatchEntry(e["id"], e["tokens"], e.get("want", [])) for e in step.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                arr.astype("<f4").tofile(os.path.join(args.out, f"{step['step']}.f32"))
            else:
                torch.cuda.current_stream().synchronize()
        for rid in step.get("end", []):
            runner.finish(rid)
        print(f"done {step['step']}", flush=True)
    return 0
