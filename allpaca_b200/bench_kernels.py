"""Times one kernel in isolation, cold in L2, and prints its rate against the roofline.

    python -m allpaca_b200.bench_kernels gemm --m 8 --n 6144 --k 4096 [--splits S] [--partials] [--swiglu]
    python -m allpaca_b200.bench_kernels attention --batch 8 --context 4096
    python -m allpaca_b200.bench_kernels prefill-attention --tokens 2048

Each call works on the next of several copies of its large operand (together larger than
the 126 MB L2), so every timed launch reads its bytes from HBM.  Times are CUDA events
around ``--iters`` launches after ``--warmup``.  This is the command the summaries under
``profiles/`` were made with (under ``ncu`` with a small ``--iters``).
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def _time(fn, iters: int, warmup: int, graph: bool = True) -> float:
    """Microseconds per launch.  The launches are recorded into one CUDA graph and replayed,
    so that the host's launch rate does not bound what is measured."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(warmup + i)
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        stop.record()
    else:
        start.record()
        for i in range(iters):
            fn(warmup + i)
        stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / iters


def bench_gemm(args) -> dict:
    from allpaca_b200 import ops
    M, N, K = args.m, args.n, args.k
    copies = max(2, int(math.ceil(300e6 / (N * K * 2))))
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    S = args.splits or ops.gemm_tc_splits(M, N, K)
    odt = torch.float32 if args.out == "float32" else torch.bfloat16
    kernel = "gemm_tc"
    if M > 64 and not args.dual and not args.single and (S == 1 or args.whole_tiles):
        # the persistent kernel; with --swiglu the rows of w alternate gate and up
        kernel = "gemm_tc_persistent"
        out = torch.empty(M, N // 2 if args.swiglu else N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_persistent(a, ws[i % copies], out, pairs=args.swiglu,   # noqa: E731
                                              share_tiles=not args.whole_tiles)
        S = 1
    elif args.dual:
        # two weight tiles per CTA; with --swiglu w is [gate; up]
        kernel = "gemm_tc_dual"
        out = torch.empty(M, N // 2 if args.swiglu else N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_dual(a, ws[i % copies], out, swiglu=args.swiglu)   # noqa: E731
        S = 1
    elif args.swiglu:
        # up to 256 rows: the gated activation in the epilogue of the (cluster) kernel
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        fn = lambda i: ops.gemm_tc(a, ws[i % copies], out, S, reduce=S > 1, pairs=True)      # noqa: E731
    elif args.partials and S > 1:
        out = torch.empty(S, M, N, device="cuda", dtype=torch.float32)
        fn = lambda i: ops.gemm_tc(a, ws[i % copies], out, S, reduce=False)      # noqa: E731
    else:
        out = torch.empty(M, N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc(a, ws[i % copies], out, S, reduce=S > 1)       # noqa: E731
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    ops.check_kernel_status()
    nbytes = N * K * 2 + M * K * 2 + out.numel() * out.element_size()
    flops = 2.0 * M * N * K
    return {"kernel": kernel, "M": M, "N": N, "K": K, "splits": S, "partials": bool(args.partials),
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 1)}


def _paged(batch, context, nkv, hd, P, scattered=False):
    """A cache and block tables: pages in rising order, as a fresh pool hands them out, or
    scattered over the pool (the worst case: one load per page)."""
    pages_per = -(-context // P)
    cache = torch.randn(batch * pages_per, 2, nkv, P, hd, device="cuda", dtype=torch.bfloat16)
    order = torch.randperm(batch * pages_per, device="cuda") if scattered else \
        torch.arange(batch * pages_per, device="cuda")
    return cache, order.to(torch.int32).view(batch, pages_per)


def bench_attention(args) -> dict:
    from allpaca_b200 import ops
    if args.splits:
        forced = args.splits
        ops.decode_splits = lambda *a, **k: forced          # try a slice count other than the plan's
    B, C, nh, nkv, hd, P = args.batch, args.context, args.heads, args.kv_heads, args.head_dim, args.page_size
    per = B * C * 2 * nkv * hd * 2
    copies = max(2, int(math.ceil(300e6 / per)))
    caches = [_paged(B, C, nkv, hd, P, args.scattered_pages) for _ in range(copies)]
    q = torch.randn(B, nh * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    seq = torch.arange(B, device="cuda", dtype=torch.int32)
    start = torch.arange(B + 1, device="cuda", dtype=torch.int32)
    pos = torch.full((B,), C - 1, device="cuda", dtype=torch.int32)
    bufs = {}

    def scratch(name, shape, dtype):
        key = (name, tuple(shape))
        if key not in bufs:
            bufs[key] = torch.empty(shape, device="cuda", dtype=dtype)
        return bufs[key]

    zeroed = {}

    def zero_scratch(name, shape, dtype):
        key = (name, tuple(shape))
        if key not in zeroed:
            zeroed[key] = torch.zeros(shape, device="cuda", dtype=dtype)
        return zeroed[key]

    def fn(i):
        cache, table = caches[i % copies]
        ops.attention(q, out, cache, table, seq, pos, nh, nkv, hd, 1.0 / math.sqrt(hd), 0, seq_start=start,
                      query_lens=[1] * B, max_context=C, scratch=scratch,
                      zero_scratch=zero_scratch if args.fused_merge else None, use_tma=not args.cp_async)
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    return {"kernel": "attention_split+merge" if args.cp_async else "attention_split_tma+merge", "batch": B, "context": C, "heads": nh, "kv_heads": nkv,
            "head_dim": hd, "splits": ops.decode_splits(B, nh, nkv, C, slots=444 if args.cp_async else 296,
                                        cluster_sizes=() if args.cp_async else (2, 4, 8, 16)),
            "us": round(us, 2),
            "GBps": round(per / us / 1e3, 1)}


def bench_prefill_attention(args) -> dict:
    from allpaca_b200 import ops
    T, nh, nkv, hd, P = args.tokens, args.heads, args.kv_heads, args.head_dim, args.page_size
    cache, table = _paged(1, T, nkv, hd, P, args.scattered_pages)
    q = torch.randn(T, nh * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    seq = torch.zeros(T, device="cuda", dtype=torch.int32)
    start = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)

    def fn(i):
        ops.attention(q, out, cache, table, seq, pos, nh, nkv, hd, 1.0 / math.sqrt(hd), 0, seq_start=start,
                      query_lens=[T], max_context=T, use_tcgen05=not args.mma_sync,
                      wide={"auto": None, "one": False, "two": True}[args.query_tiles])
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    flops = 4.0 * nh * hd * T * (T + 1) / 2
    return {"kernel": "attention_tile" if args.mma_sync else "attention_tcgen05", "query_tiles": args.query_tiles, "tokens": T, "heads": nh, "kv_heads": nkv, "head_dim": hd,
            "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m allpaca_b200.bench_kernels")
    sub = p.add_subparsers(dest="what", required=True)
    for name in ("gemm", "attention", "prefill-attention"):
        s = sub.add_parser(name)
        s.add_argument("--iters", type=int, default=50)
        s.add_argument("--warmup", type=int, default=5)
        s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
        if name == "gemm":
            s.add_argument("--m", type=int, default=8)
            s.add_argument("--n", type=int, default=4096)
            s.add_argument("--k", type=int, default=4096)
            s.add_argument("--splits", type=int, default=0, help="K slices (0: the kernel's own plan)")
            s.add_argument("--partials", action="store_true", help="write partial sums instead of adding in a cluster")
            s.add_argument("--out", choices=["float32", "bfloat16"], default="bfloat16")
            s.add_argument("--dual", action="store_true", help="more than 64 rows: two weight tiles per CTA")
            s.add_argument("--single", action="store_true", help="more than 64 rows: one tile per CTA, not persistent")
            s.add_argument("--whole-tiles", action="store_true",
                           help="persistent kernel: never share a tile's K among several CTAs")
            s.add_argument("--swiglu", action="store_true", help="w holds gate and up rows: fused gated activation")
        else:
            s.add_argument("--heads", type=int, default=32)
            s.add_argument("--kv-heads", type=int, default=8)
            s.add_argument("--head-dim", type=int, default=128)
            s.add_argument("--page-size", type=int, default=16)
            s.add_argument("--batch", type=int, default=8)
            s.add_argument("--context", type=int, default=4096)
            s.add_argument("--tokens", type=int, default=2048)
            s.add_argument("--fused-merge", action="store_true",
                           help="cp.async kernel: the last slice to arrive combines them all")
            s.add_argument("--cp-async", action="store_true", help="decode: the cp.async kernel instead of the TMA one")
            s.add_argument("--splits", type=int, default=0, help="key slices (0: the kernel's own plan)")
            s.add_argument("--mma-sync", action="store_true", help="prompt attention with the mma.sync tile kernel")
            s.add_argument("--query-tiles", choices=["auto", "one", "two"], default="auto",
                           help="prompt attention on tcgen05: query tiles to a CTA (auto: by the number of CTAs)")
            s.add_argument("--scattered-pages", action="store_true",
                           help="block tables in random order instead of rising page numbers")
    args = p.parse_args(argv)
    fn = {"gemm": bench_gemm, "attention": bench_attention, "prefill-attention": bench_prefill_attention}[args.what]
    print(json.dumps(fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
