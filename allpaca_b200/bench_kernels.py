"""Times one kernel in isolation, cold in L2, and prints its rate against the roofline.

    python -m allpaca_b200.bench_kernels gemm --m 8 --n 6144 --k 4096 [--splits S] [--partials] [--swiglu]
    python -m allpaca_b200.bench_kernels attention --batch 8 --context 4096
    python -m allpaca_b200.bench_kernels prefill-attention --tokens 2048
    python -m allpaca_b200.bench_kernels versus-reference      # a table: ours against the reference's own kernels

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
    if (M > 128 and not args.dual and not args.pair and not args.single and (S == 1 or args.whole_tiles)) \
            or args.persistent:
        # the persistent kernel; with --swiglu the rows of w alternate gate and up
        kernel = "gemm_tc_persistent"
        out = torch.empty(M, N // 2 if args.swiglu else N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_persistent(a, ws[i % copies], out, pairs=args.swiglu,   # noqa: E731
                                              share_tiles=not args.whole_tiles)
        S = 1
    elif args.pair:
        # a pair of CTAs to a tile of 256 weight rows (cta_group::2); with --swiglu the rows of w alternate
        kernel = "gemm_tc_pair"
        out = torch.empty(M, N // 2 if args.swiglu else N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_pair(a, ws[i % copies], out, pairs=args.swiglu,   # noqa: E731
                                        share_tiles=not args.whole_tiles)
        S = 1
    elif args.dual:
        # two weight tiles per CTA
        kernel = "gemm_tc_dual"
        out = torch.empty(M, N, device="cuda", dtype=odt)
        fn = lambda i: ops.gemm_tc_dual(a, ws[i % copies], out)   # noqa: E731
        S = 1
    elif args.residual:
        # few rows: the product adds into the 32-bit residual, writes its bfloat16 copy and the
        # partial sums of squares of its rows (the epilogue of the O and down products of a decode step)
        kernel = "gemm_tc (residual epilogue)"
        out = torch.randn(M, N, device="cuda", dtype=torch.float32)
        xb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ss = torch.empty(M, ops.gemm_tc_residual_parts(N, S), device="cuda", dtype=torch.float32)
        fn = lambda i: ops.gemm_tc_residual(a, ws[i % copies], out, xb, ss, S)     # noqa: E731
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

    mean = C
    if args.short_context:
        # one long sequence among short ones
        pos[1:] = args.short_context - 1
        mean = (C + (B - 1) * args.short_context) // B
        per = per * mean // C

    def fn(i):
        cache, table = caches[i % copies]
        ops.attention(q, out, cache, table, seq, pos, nh, nkv, hd, 1.0 / math.sqrt(hd), 0, seq_start=start,
                      query_lens=[1] * B, max_context=C, scratch=scratch, use_tma=not args.cp_async,
                      mean_context=0 if args.plan_by_longest else mean)
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    return {"kernel": "attention_split+merge" if args.cp_async else "attention_split_tma+merge", "batch": B, "context": C, "heads": nh, "kv_heads": nkv,
            "head_dim": hd, "mean_context": mean,
            "splits": ops.decode_splits(B, nh, nkv, C, slots=444 if args.cp_async else 296,
                                        cluster_sizes=() if args.cp_async else (2, 4, 8, 16),
                                        mean_context=0 if args.plan_by_longest else mean),
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


def bench_versus_reference(args) -> dict:
    """The operations of a decode step at the Llama-3.1-8B sizes (8 rows; 2048 keys), and the prompt
    attention of 512 tokens: the reference's own CUDA kernels (32-bit float, its only precision;
    ``baseline/reference_kernels.py``) against this engine's kernel of the same operation in 32-bit
    and in bfloat16 (what serving runs).  Launched from the host one after the other, CUDA events
    around ``--iters`` launches; large operands rotate over copies that together exceed L2."""
    import os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from allpaca_b200 import ops
    from baseline import reference_kernels
    ref = reference_kernels.load()
    if ref is None:
        return {"unavailable": "the reference's kernels are not built here"}
    H, NH, NKV, HD, INTER, M, KEYS = 4096, 32, 8, 128, 14336, 8, 2048
    rows = []

    def timed(fn):
        return round(_time(fn, args.iters, args.warmup, graph=False), 2)

    def weights(n, k, dtype):
        copies = max(2, int(math.ceil(300e6 / (n * k * torch.empty((), dtype=dtype).element_size()))))
        return [(torch.randn(n, k, device="cuda") * 0.02).to(dtype) for _ in range(min(copies, 8))]

    for name, n, k in (("QKV product", (NH + 2 * NKV) * HD, H), ("O product", H, NH * HD),
                       ("gate and up products + SiLU*up", 2 * INTER, H), ("down product", H, INTER)):
        w32 = weights(n, k, torch.float32)
        a32 = torch.randn(M, k, device="cuda")
        out32 = torch.empty(M, n, device="cuda")
        if name.startswith("gate"):
            act = torch.empty(M, INTER, device="cuda")

            g32, u32 = torch.empty(M, INTER, device="cuda"), torch.empty(M, INTER, device="cuda")

            def theirs(i):
                w = w32[i % len(w32)]
                ref.gemm_nt(a32, w[:INTER], g32)
                ref.gemm_nt(a32, w[INTER:], u32)
                ref.silu_mul(g32, u32, act)

            def ours32(i):
                ops.gemm_simt(a32, w32[i % len(w32)], out32)
                ops.swiglu(out32, act)
        else:
            def theirs(i):
                ref.gemm_nt(a32, w32[i % len(w32)], out32)

            def ours32(i):
                ops.gemm_simt(a32, w32[i % len(w32)], out32)
        t_ref, t32 = timed(theirs), timed(ours32)
        del w32
        w16 = weights(n, k, torch.bfloat16)
        a16 = a32.bfloat16()
        S = ops.gemm_tc_splits(M, n, k)
        if name.startswith("gate"):
            out16 = torch.empty(M, INTER, device="cuda", dtype=torch.bfloat16)

            def ours16(i):
                ops.gemm_tc(a16, w16[i % len(w16)], out16, S, reduce=S > 1, pairs=True)
        else:
            out16 = torch.empty(M, n, device="cuda", dtype=torch.bfloat16)

            def ours16(i):
                ops.gemm_tc(a16, w16[i % len(w16)], out16, S, reduce=S > 1)
        rows.append((f"{name}, {M} x {n} x {k}", t_ref, t32, timed(ours16)))
        del w16
    # norm
    x, w = torch.randn(M, H, device="cuda"), torch.ones(H, device="cuda")
    o32, o16 = torch.empty(M, H, device="cuda"), torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    rows.append((f"RMSNorm, {M} x {H}", timed(lambda i: ref.rmsnorm_rows(x, w, o32, 1e-5)),
                 timed(lambda i: ops.add_rmsnorm(x, w, 1e-5, o32)), timed(lambda i: ops.add_rmsnorm(x, w, 1e-5, o16))))
    # rotation of 8 rows at one position each (the reference: one launch per row, as its decode does)
    q, k = torch.randn(M, NH, HD, device="cuda"), torch.randn(M, NKV, HD, device="cuda")
    qkv = torch.randn(M, (NH + 2 * NKV) * HD, device="cuda")
    pos = torch.arange(100, 100 + M, device="cuda", dtype=torch.int32)
    inv = torch.rand(HD // 2, device="cuda")
    table = torch.empty(M, HD // 2, 2, device="cuda")
    q_out32 = torch.empty(M, NH * HD, device="cuda")
    q_out16 = torch.empty(M, NH * HD, device="cuda", dtype=torch.bfloat16)
    qkv16 = qkv.bfloat16()

    def their_rope(i):
        for r in range(M):
            ref.rope_adjacent(q[r:r + 1], k[r:r + 1], 100 + r, 500000.0)

    def our_rope(out, src):
        def fn(i):
            ops.rope_table(pos, inv, table)
            ops.rope_kv_store(src, out, None, pos, None, None, table, 0, NH, NKV, HD)
        return fn
    rows.append((f"rotation of Q and K, {M} rows", timed(their_rope), timed(our_rope(q_out32, qkv)),
                 timed(our_rope(q_out16, qkv16))))
    # decode attention: 8 sequences of 2048 keys (the reference: one call per sequence)
    kk, vv = torch.randn(M, KEYS, NKV, HD, device="cuda"), torch.randn(M, KEYS, NKV, HD, device="cuda")
    qd = torch.randn(M, 1, NH, HD, device="cuda")
    od = torch.empty_like(qd)

    def their_decode(i):
        for b in range(M):
            ref.attention(qd[b], kk[b], vv[b], od[b], causal=True)
    P = 16
    seq = torch.arange(M, device="cuda", dtype=torch.int32)
    start = torch.arange(M + 1, device="cuda", dtype=torch.int32)
    last = torch.full((M,), KEYS - 1, device="cuda", dtype=torch.int32)
    bufs = {}

    def scratch(name, shape, dtype):
        return bufs.setdefault((name, tuple(shape)), torch.empty(shape, device="cuda", dtype=dtype))

    def our_decode(dtype):
        cache, tbl = _paged(M, KEYS, NKV, HD, P)
        cache = cache.to(dtype)
        qq = torch.randn(M, NH * HD, device="cuda").to(dtype)
        oo = torch.empty_like(qq)
        return lambda i: ops.attention(qq, oo, cache, tbl, seq, last, NH, NKV, HD, HD ** -0.5, 0, seq_start=start,
                                       query_lens=[1] * M, max_context=KEYS, scratch=scratch)
    rows.append((f"decode attention, {M} sequences x {KEYS} keys", timed(their_decode),
                 timed(our_decode(torch.float32)), timed(our_decode(torch.bfloat16))))
    # prompt attention of 512 tokens
    T = 512
    qp, kp, vp = (torch.randn(T, n, HD, device="cuda") for n in (NH, NKV, NKV))
    op = torch.empty_like(qp)

    def our_prompt(dtype):
        cache, tbl = _paged(1, T, NKV, HD, P)
        cache = cache.to(dtype)
        qq = torch.randn(T, NH * HD, device="cuda").to(dtype)
        oo = torch.empty_like(qq)
        ts = torch.zeros(T, device="cuda", dtype=torch.int32)
        st = torch.tensor([0, T], device="cuda", dtype=torch.int32)
        ps = torch.arange(T, device="cuda", dtype=torch.int32)
        return lambda i: ops.attention(qq, oo, cache, tbl, ts, ps, NH, NKV, HD, HD ** -0.5, 0, seq_start=st,
                                       query_lens=[T], max_context=T)
    rows.append((f"prompt attention, {T} tokens, causal", timed(lambda i: ref.attention(qp, kp, vp, op, causal=True)),
                 timed(our_prompt(torch.float32)), timed(our_prompt(torch.bfloat16))))
    ops.check_kernel_status()
    print("| operation | reference kernel (32-bit), us | ours 32-bit, us | ours bfloat16, us | reference / ours bfloat16 |")
    print("|---|---|---|---|---|")
    for name, a, b, c in rows:
        print(f"| {name} | {a} | {b} | {c} | {a / c:.1f}x |")
    return {"rows": [{"operation": n, "reference_us": a, "ours_float32_us": b, "ours_bfloat16_us": c} for n, a, b, c in rows]}


def bench_sampling(args) -> dict:
    """The choice of the next token for ``--rows`` rows of logits over ``--vocab`` entries."""
    from allpaca_b200 import ops
    R, V = args.rows, args.vocab
    copies = max(2, int(math.ceil(300e6 / (R * V * 4))))
    logits = [torch.randn(R, V, device="cuda") * args.spread for _ in range(copies)]
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    temp = torch.full((R,), args.temperature, device="cuda")
    top_k = torch.full((R,), args.top_k, dtype=torch.int32, device="cuda")
    top_p = torch.full((R,), args.top_p, device="cuda")
    uniform = torch.rand(R, device="cuda")
    if args.temperature <= 1e-5:
        kernel, fn = "argmax", (lambda i: ops.argmax(logits[i % copies], out))     # noqa: E731
    else:
        kernel = "sample"
        fn = lambda i: ops.sample(logits[i % copies], temp, top_k, top_p, uniform, out)   # noqa: E731
    us = _time(fn, args.iters, args.warmup, not args.no_graph)
    return {"kernel": kernel, "rows": R, "vocab": V, "temperature": args.temperature, "top_k": args.top_k,
            "top_p": args.top_p, "us": round(us, 2), "GBps": round(R * V * 4 / us / 1e3, 1)}


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
            s.add_argument("--pair", action="store_true", help="more than 64 rows: a pair of CTAs to a tile (cta_group::2)")
            s.add_argument("--single", action="store_true", help="more than 64 rows: one tile per CTA, not persistent")
            s.add_argument("--persistent", action="store_true", help="the persistent kernel, whatever the plan says")
            s.add_argument("--whole-tiles", action="store_true",
                           help="persistent and pair kernel: never share a tile's K among several CTAs")
            s.add_argument("--swiglu", action="store_true", help="w holds gate and up rows: fused gated activation")
            s.add_argument("--residual", action="store_true",
                           help="few rows: add into a 32-bit residual in the epilogue (with its bfloat16 copy and sums of squares)")
        else:
            s.add_argument("--heads", type=int, default=32)
            s.add_argument("--kv-heads", type=int, default=8)
            s.add_argument("--head-dim", type=int, default=128)
            s.add_argument("--page-size", type=int, default=16)
            s.add_argument("--batch", type=int, default=8)
            s.add_argument("--context", type=int, default=4096)
            s.add_argument("--tokens", type=int, default=2048)
            s.add_argument("--cp-async", action="store_true", help="decode: the cp.async kernel instead of the TMA one")
            s.add_argument("--short-context", type=int, default=0,
                           help="decode: every sequence but the first holds this many keys (0: all hold --context)")
            s.add_argument("--plan-by-longest", action="store_true",
                           help="decode: plan the key slices as if every sequence were as long as the longest")
            s.add_argument("--splits", type=int, default=0, help="key slices (0: the kernel's own plan)")
            s.add_argument("--mma-sync", action="store_true", help="prompt attention with the mma.sync tile kernel")
            s.add_argument("--query-tiles", choices=["auto", "one", "two"], default="auto",
                           help="prompt attention on tcgen05: query tiles to a CTA (auto: by the number of CTAs)")
            s.add_argument("--scattered-pages", action="store_true",
                           help="block tables in random order instead of rising page numbers")
    s = sub.add_parser("sampling")
    s.add_argument("--iters", type=int, default=50)
    s.add_argument("--warmup", type=int, default=5)
    s.add_argument("--no-graph", action="store_true", help="launch from the host (for ncu)")
    s.add_argument("--rows", type=int, default=8)
    s.add_argument("--vocab", type=int, default=128256)
    s.add_argument("--temperature", type=float, default=0.8, help="0: the arg-max kernel")
    s.add_argument("--top-k", type=int, default=40, help="0: off")
    s.add_argument("--top-p", type=float, default=0.95, help="1: off")
    s.add_argument("--spread", type=float, default=3.0, help="standard deviation of the random logits")
    s = sub.add_parser("versus-reference")
    s.add_argument("--iters", type=int, default=20)
    s.add_argument("--warmup", type=int, default=3)
    args = p.parse_args(argv)
    fn = {"gemm": bench_gemm, "attention": bench_attention, "prefill-attention": bench_prefill_attention,
          "sampling": bench_sampling, "versus-reference": bench_versus_reference}[args.what]
    print(json.dumps(fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
