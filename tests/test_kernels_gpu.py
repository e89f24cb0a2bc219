"""Each CUDA kernel alone against a plain float32/float64 torch reference of the same
operation, at sizes other than the engine's (odd widths, tails, head sizes in steps of 16)."""
import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from allpaca_b200 import ops as o
    return o


def dev(t):
    return t.to("cuda")


def rel_err(got, ref):
    ref = ref.double()
    return float((got.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


# ---------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(301, 120, generator=g).to(dtype)
    tokens = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32)
    x = torch.empty(5, 120, dtype=torch.float32, device="cuda")
    ops.embed_gather(dev(tokens), dev(table), x)
    assert torch.equal(x.cpu(), table[tokens.long()].float())


# ---------------------------------------------------------------- norm
@pytest.mark.parametrize("H", [64, 120, 4096, 13001])
@pytest.mark.parametrize("S", [0, 1, 3])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(ops, H, S, out_dtype):
    g = torch.Generator().manual_seed(H + S)
    T = 5
    x = torch.randn(T, H, generator=g) * 3
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(out_dtype)
    delta = torch.randn(max(S, 1), T, H, generator=g) if S else None
    eps = 1e-6 if H % 2 else 1e-5
    xd = dev(x.clone())
    out = torch.empty(T, H, dtype=out_dtype, device="cuda")
    ops.add_rmsnorm(xd, dev(w), eps, out, delta=dev(delta) if S else None)
    v = x.double() + (delta.double().sum(0) if S else 0)
    ref = plain_llama.rmsnorm(v, w.double(), eps)
    assert rel_err(xd.cpu(), v) < 1e-6                     # the residual is updated in 32-bit
    assert rel_err(out.cpu(), ref) < (1e-5 if out_dtype == torch.float32 else 5e-3)
    # chosen rows only: x is left alone
    rows = torch.tensor([4, 0, 2], dtype=torch.int32)
    xd2 = dev(x.clone())
    out2 = torch.empty(3, H, dtype=out_dtype, device="cuda")
    ops.add_rmsnorm(xd2, dev(w), eps, out2, delta=dev(delta) if S else None, rows=dev(rows))
    assert torch.equal(xd2.cpu(), x)
    assert rel_err(out2.cpu(), ref[rows.long()]) < (1e-5 if out_dtype == torch.float32 else 5e-3)


def test_residual_add(ops):
    x = torch.randn(7, 33)
    d = torch.randn(2, 7, 33)
    xd = dev(x.clone())
    ops.residual_add(xd, dev(d))
    assert rel_err(xd.cpu(), x.double() + d.double().sum(0)) < 1e-6


# ---------------------------------------------------------------- rotary + cache write
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,P", [(4, 2, 16, 16), (3, 1, 32, 8), (6, 3, 48, 4), (5, 5, 80, 16)])
def test_rope_kv_store(ops, dtype, nh, nkv, hd, P):
    from allpaca_b200.parts.rope import inverse_frequencies
    g = torch.Generator().manual_seed(hd)
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64} if hd == 32 else None
    inv = inverse_frequencies(hd, 500000.0 if scaling else 10000.0, scaling)
    ref_inv = plain_llama.rope_inverse_frequencies(
        hd, 500000.0 if scaling else 10000.0,
        dict(scaling, rope_type="llama3") if scaling else None)
    assert torch.allclose(inv, ref_inv, rtol=1e-12, atol=0)
    # two sequences: rows 0..4 are positions 3..7 of sequence 0, rows 5..6 positions 20..21 of sequence 1
    positions = torch.tensor([3, 4, 5, 6, 7, 20, 21], dtype=torch.int32)
    token_seq = torch.tensor([0, 0, 0, 0, 0, 1, 1], dtype=torch.int32)
    T = 7
    n_pages = 12
    table = torch.full((2, 8), -1, dtype=torch.int32)
    table[0, :3] = torch.tensor([5, 2, 9])
    table[1, :6] = torch.tensor([0, 1, 3, 4, 6, 7])
    width = (nh + 2 * nkv) * hd
    S = 2 if dtype == torch.float32 else 1
    qkv = torch.randn(S, T, width, generator=g)
    inp = qkv if dtype == torch.float32 else qkv[0].to(dtype)
    cache = torch.zeros(n_pages, 2, nkv, P, hd, dtype=dtype)
    cd = dev(cache)
    q_out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
    cos_sin = torch.empty(T, hd // 2, 2, device="cuda")
    ops.rope_table(dev(positions), dev(inv.float()), cos_sin)
    ops.rope_kv_store(dev(inp), q_out, cd, dev(positions), dev(token_seq), dev(table),
                      cos_sin, 0, nh, nkv, hd)
    full = (qkv.sum(0) if dtype == torch.float32 else inp.float()).double()
    q = full[:, :nh * hd].view(T, nh, hd)
    k = full[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = full[:, (nh + nkv) * hd:].view(T, nkv, hd)
    tol = 2e-5 if dtype == torch.float32 else 6e-3
    qr = plain_llama.rope_half_split(q, positions, inv)
    kr = plain_llama.rope_half_split(k, positions, inv)
    assert rel_err(q_out.cpu().view(T, nh, hd), qr) < tol
    got = cd.cpu()
    touched = torch.zeros(n_pages, P, dtype=torch.bool)
    for t in range(T):
        pos, s = int(positions[t]), int(token_seq[t])
        page = int(table[s, pos // P])
        touched[page, pos % P] = True
        assert rel_err(got[page, 0, :, pos % P, :], kr[t]) < tol
        assert rel_err(got[page, 1, :, pos % P, :], v[t]) < tol
    # nothing else in the cache was written
    assert float(got[:, :, :, :, :].abs().sum(dim=(1, 2, 4))[~touched].sum()) == 0.0


def test_rope_adjacent_pairing_and_no_rotation(ops):
    nh, hd, T = 2, 16, 3
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, nh * hd, generator=g)
    positions = torch.tensor([0, 5, 9], dtype=torch.int32)
    inv = plain_llama.rope_inverse_frequencies(hd, 10000.0, None)
    out = torch.empty(T, nh * hd, device="cuda")
    cos_sin = torch.empty(T, hd // 2, 2, device="cuda")
    ops.rope_table(dev(positions), dev(inv.float()), cos_sin)
    ops.rope_kv_store(dev(x), out, None, dev(positions), None, None, cos_sin, 1, nh, 0, hd)
    xv = x.double().view(T, nh, hd // 2, 2)
    ang = positions.double()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    ref = torch.stack([xv[..., 0] * c - xv[..., 1] * s, xv[..., 0] * s + xv[..., 1] * c], -1)
    assert rel_err(out.cpu().view(T, nh, hd // 2, 2), ref) < 2e-5
    ops.rope_kv_store(dev(x), out, None, dev(positions), None, None, None, 0, nh, 0, hd)
    assert torch.equal(out.cpu(), x)


# ---------------------------------------------------------------- gated activation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [177, 200])
@pytest.mark.parametrize("pairs", [False, True])
def test_swiglu(ops, dtype, I, pairs):
    g = torch.Generator().manual_seed(2)
    T = 5
    S = 3 if dtype == torch.float32 else 1
    gu = torch.randn(S, T, 2 * I, generator=g) * 2
    inp = gu if dtype == torch.float32 else gu[0].to(dtype)
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    ops.swiglu(dev(inp), out, pairs=pairs)
    full = (gu.sum(0) if dtype == torch.float32 else inp.float()).double()
    gate, up = (full[:, 0::2], full[:, 1::2]) if pairs else (full[:, :I], full[:, I:])
    ref = plain_llama.silu(gate) * up
    assert rel_err(out.cpu(), ref) < (1e-5 if dtype == torch.float32 else 5e-3)


# ---------------------------------------------------------------- matrix products
SHAPES = [(1, 64, 64), (5, 176, 64), (8, 301, 120), (33, 96, 256), (64, 130, 200), (100, 257, 72),
          (130, 512, 136), (300, 640, 1000)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_simt_float32_is_true_32_bit(ops, M, N, K):
    g = torch.Generator().manual_seed(M)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = torch.empty(M, N, device="cuda")
    ops.gemm_simt(dev(a), dev(w), out)
    ref = a.double() @ w.double().T
    # a reduced-precision operand mode (tf32, bf16) would be off by 1e-3; true 32-bit is ~1e-6
    assert rel_err(out.cpu(), ref) < 3e-6


@pytest.mark.parametrize("M,N,K", SHAPES[:5])
@pytest.mark.parametrize("wdtype,odtype", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                           (torch.float32, torch.bfloat16), (torch.float32, torch.float32)])
def test_gemm_simt_bfloat16(ops, M, N, K, wdtype, odtype):
    g = torch.Generator().manual_seed(M)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).to(wdtype)
    out = torch.empty(M, N, dtype=odtype, device="cuda")
    ops.gemm_simt(dev(a), dev(w), out)
    ref = a.double() @ w.double().T
    assert rel_err(out.cpu(), ref) < (3e-6 if odtype == torch.float32 else 5e-3)


TC_SHAPES = [(1, 128, 64), (3, 64, 64), (8, 301, 120), (16, 256, 512), (17, 130, 200), (40, 640, 4096),
             (64, 384, 1024), (100, 257, 72), (128, 512, 136), (200, 128, 64), (256, 1000, 320),
             (300, 640, 1000), (700, 384, 2048)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_gemm_tensor_cores(ops, M, N, K, odtype):
    assert ops.tensor_core_gemm_available()
    g = torch.Generator().manual_seed(N + K)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).bfloat16()
    out = torch.full((M + 2, N), 7.0, dtype=odtype, device="cuda")       # two guard rows
    ops.gemm_tc(dev(a), dev(w), out[:M], 1)
    ops.check_kernel_status()
    ref = a.double() @ w.double().T
    assert rel_err(out[:M].cpu(), ref) < (1e-5 if odtype == torch.float32 else 5e-3)
    assert torch.all(out[M:] == 7.0)                                       # nothing written past M


@pytest.mark.parametrize("M,N,K,S", [(1, 128, 512, 2), (8, 301, 1000, 3), (16, 256, 4096, 8),
                                     (64, 384, 1024, 4), (5, 640, 14336, 16)])
def test_gemm_tensor_cores_split_k(ops, M, N, K, S):
    g = torch.Generator().manual_seed(S)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).bfloat16()
    out = torch.empty(S, M, N, dtype=torch.float32, device="cuda")
    ops.gemm_tc(dev(a), dev(w), out, S)
    ops.check_kernel_status()
    ref = a.double() @ w.double().T
    assert rel_err(out.sum(0).cpu(), ref) < 1e-5
    planned = ops.gemm_tc_splits(M, N, K)
    kb = -(-K // 64)
    assert 1 <= planned <= kb and (planned - 1) * (-(-kb // planned)) < kb


def test_gemm_tensor_cores_refuses_what_tma_cannot_take(ops):
    a = torch.randn(4, 68).bfloat16().cuda()
    w = torch.randn(8, 68).bfloat16().cuda()
    out = torch.empty(4, 8, dtype=torch.float32, device="cuda")
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.gemm_tc(a, w, out, 1)


# ---------------------------------------------------------------- sampling
def test_argmax_first_maximum(ops):
    logits = torch.randn(6, 1000)
    logits[2, 17] = logits[2, 400] = 50.0          # tie: the lower id wins
    logits[3, :] = float("-inf")                    # nothing finite: token 0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(dev(logits), out)
    want = [int(torch.argmax(r)) for r in logits]
    want[2], want[3] = 17, 0
    assert out.cpu().tolist() == want


def check_samples(ops, logits, cases, method):
    """``cases``: (temperature, top_k, top_p, uniform) per row of ``logits``."""
    R = len(cases)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(torch.tensor([c[0] for c in cases])),
               dev(torch.tensor([c[1] for c in cases], dtype=torch.int32)),
               dev(torch.tensor([c[2] for c in cases])), dev(torch.tensor([c[3] for c in cases])), out,
               method=method)
    got = out.cpu().tolist()
    for r, (temp, k, p, u) in enumerate(cases):
        want = plain_llama.sample_plain(logits[r], temp, k, p, u)
        if got[r] != want:
            # allowed only when u sits on a boundary of the cumulative distribution (rounding)
            alt = {plain_llama.sample_plain(logits[r], temp, k, p, min(max(u + d, 0.0), 0.999999))
                   for d in (-2e-6, 2e-6)}
            assert got[r] in alt, (r, cases[r], got[r], want)


@pytest.mark.parametrize("method", ["cluster", "rows"])
@pytest.mark.parametrize("V", [64, 301, 5000])
def test_sample_matches_plain(ops, V, method):
    g = torch.Generator().manual_seed(V)
    cases = []
    for temp, k, p in [(0.0, 0, 1.0), (0.8, 0, 1.0), (1.3, 5, 1.0), (0.7, 0, 0.9), (0.8, 40, 0.95),
                       (1.0, 1, 0.5), (2.0, 10, 0.0), (0.5, 1000000, 0.3)]:
        for u in (0.0, 0.25, 0.5, 0.99):
            cases.append((temp, k, p, u))
    R = len(cases)
    logits = torch.randn(R, V, generator=g) * 2
    logits[5, 3] = logits[5, 9] = logits[5].max() + 1      # ties at the top
    logits[7, ::3] = float("-inf")                           # non-finite entries are dropped
    check_samples(ops, logits, cases, method)


@pytest.mark.parametrize("method", ["cluster", "rows"])
def test_sample_where_many_logits_are_equal_or_far_away(ops, method):
    """Rows that defeat a search by value: thousands of equal logits at the cut (more than the
    sorted list of the cluster kernel holds), a few logits far below the rest, a single finite
    logit, and a row of two values only."""
    V = 6000
    g = torch.Generator().manual_seed(11)
    rows, cases = [], []

    def add(row, temp, k, p, us=(0.0, 0.3, 0.77, 0.999)):
        for u in us:
            rows.append(row.clone())
            cases.append((temp, k, p, u))
    flat = torch.zeros(V)
    add(flat, 1.0, 0, 1.0)
    add(flat, 1.0, 10, 1.0)
    add(flat, 0.7, 3000, 1.0)
    add(flat, 1.0, 0, 0.5003)            # (not 0.5: 3000 equal shares would reach it up to rounding only)
    add(flat, 1.0, 4000, 0.9003)
    two = torch.zeros(V)
    two[::2] = 1.5                       # 3000 equal logits above 3000 equal ones
    add(two, 1.0, 3500, 1.0)
    add(two, 1.0, 2500, 0.7003)
    add(two, 0.9, 0, 0.95)
    far = torch.randn(V, generator=g)
    far[100:130] = -1e9                  # masked out by a large negative number
    far[7] = -3e38
    add(far, 0.8, 40, 0.95)
    add(far, 0.8, V - 5, 1.0)            # the cut lies among the far ones
    add(far, 1.2, 0, 0.999)
    lone = torch.full((V,), float("-inf"))
    lone[4321] = 0.25
    add(lone, 0.8, 40, 0.95)
    add(lone, 0.8, 0, 0.2)
    check_samples(ops, torch.stack(rows), cases, method)


@pytest.mark.parametrize("V", [128256, 200003])
def test_sample_large_vocabulary(ops, V):
    """The cluster kernel at the sizes it is for (32 and 64 logits a thread), against the plain
    sampler on a few rows and against the kernel with one CTA per row on all of them."""
    g = torch.Generator().manual_seed(V)
    settings = [(0.8, 40, 0.95), (0.8, 0, 1.0), (1.0, 0, 0.9), (0.6, 3000, 0.99), (1.5, 1, 1.0), (0.0, 0, 1.0),
                (0.9, 2048, 0.5), (1.0, 0, 0.0)]
    cases = [(t, k, p, u) for (t, k, p) in settings for u in (0.0, 0.41, 0.93)]
    R = len(cases)
    logits = torch.randn(R, V, generator=g) * 3
    logits[:, 1000:1010] = float("nan")
    outs = {}
    for method in ("cluster", "rows"):
        out = torch.empty(R, dtype=torch.int32, device="cuda")
        ops.sample(dev(logits), dev(torch.tensor([c[0] for c in cases])),
                   dev(torch.tensor([c[1] for c in cases], dtype=torch.int32)),
                   dev(torch.tensor([c[2] for c in cases])), dev(torch.tensor([c[3] for c in cases])), out,
                   method=method)
        outs[method] = out.cpu().tolist()
    differ = [r for r in range(R) if outs["cluster"][r] != outs["rows"][r]]
    assert len(differ) <= 1, differ          # a draw on a boundary of the cumulative distribution may differ
    check_samples(ops, logits[:4], cases[:4], "cluster")


def test_sample_distribution(ops):
    """Draws follow softmax(logits / T) restricted to the top-k."""
    V, n = 50, 20000
    g = torch.Generator().manual_seed(5)
    row = torch.randn(V, generator=g)
    temp, k = 0.9, 8
    logits = row.expand(n, V).contiguous()
    u = torch.rand(n, generator=g)
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(torch.full((n,), temp)), dev(torch.full((n,), k, dtype=torch.int32)),
               dev(torch.ones(n)), dev(u), out)
    counts = torch.bincount(out.cpu().long(), minlength=V).double()
    top = torch.topk(row, k).indices
    p = torch.zeros(V, dtype=torch.float64)
    p[top] = torch.softmax(row[top].double() / temp, 0)
    assert counts[p == 0].sum() == 0
    chi2 = float((((counts - n * p) ** 2)[p > 0] / (n * p[p > 0])).sum())
    assert chi2 < 30.0            # 7 degrees of freedom: P(chi2 > 30) ~ 1e-4


# ---------------------------------------------------------------- attention over pages
def paged_case(seqs, nh, nkv, hd, P, dtype, seed, freed_before=None, sequential=False):
    """Random queries and a paged cache for sequences given as (context length, query rows).
    Pages are handed out in a shuffled order so that neighbours in a sequence are far apart
    in memory (`sequential`: in rising order, as a fresh pool hands them out).
    `freed_before[s]`: pages wholly before that position are marked given back."""
    g = torch.Generator().manual_seed(seed)
    max_pages = max(-(-c // P) for c, _ in seqs)
    total_pages = sum(-(-c // P) for c, _ in seqs) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    if sequential:
        perm = list(range(total_pages - 1, -1, -1))          # pop() hands out 0, 1, 2, ...
    cache = torch.randn(total_pages, 2, nkv, P, hd, generator=g).to(dtype)   # junk in unused slots
    table = torch.full((len(seqs), max_pages), -1, dtype=torch.int32)
    ks, vs, rows_q, token_seq, positions, seq_start = [], [], [], [], [], [0]
    for s, (ctx, qn) in enumerate(seqs):
        k = torch.randn(ctx, nkv, hd, generator=g).to(dtype)
        v = torch.randn(ctx, nkv, hd, generator=g).to(dtype)
        for j in range(-(-ctx // P)):
            page = perm.pop()
            n = min(P, ctx - j * P)
            if freed_before and j * P + P <= freed_before[s]:
                continue                                            # given back: stays -1
            table[s, j] = page
            cache[page, 0, :, :n] = k[j * P:j * P + n].transpose(0, 1)
            cache[page, 1, :, :n] = v[j * P:j * P + n].transpose(0, 1)
        ks.append(k), vs.append(v)
        rows_q.append(torch.randn(qn, nh, hd, generator=g).to(dtype))
        token_seq += [s] * qn
        positions += list(range(ctx - qn, ctx))
        seq_start.append(seq_start[-1] + qn)
    q = torch.cat(rows_q).reshape(-1, nh * hd)
    return dict(q=q, cache=cache, table=table, token_seq=torch.tensor(token_seq, dtype=torch.int32),
                positions=torch.tensor(positions, dtype=torch.int32),
                seq_start=torch.tensor(seq_start, dtype=torch.int32), ks=ks, vs=vs, rows_q=rows_q,
                query_lens=[qn for _, qn in seqs])


def reference_attention(case, seqs, nh, hd, window, scale=None):
    outs = []
    for s, (ctx, qn) in enumerate(seqs):
        qfull = torch.zeros(ctx, nh, hd, dtype=torch.float64)
        qfull[ctx - qn:] = case["rows_q"][s].double()
        o = plain_llama.causal_attention(qfull, case["ks"][s].double(), case["vs"][s].double(),
                                         window=window, scale=scale)
        outs.append(o[ctx - qn:])
    return torch.cat(outs).reshape(-1, nh * hd)


def run_attention(ops, case, nh, nkv, hd, scale, window, tensor_cores, **more):
    q = dev(case["q"])
    out = torch.empty_like(q)
    bufs = {}

    def scratch(name, shape, dtype):
        bufs[name] = torch.empty(shape, dtype=dtype, device="cuda")
        return bufs[name]
    kw = {}
    if tensor_cores:
        kw = dict(seq_start=dev(case["seq_start"]), query_lens=case["query_lens"],
                  max_context=int(case["positions"].max()) + 1, scratch=scratch)
    ops.attention(q, out, dev(case["cache"]), dev(case["table"]), dev(case["token_seq"]),
                  dev(case["positions"]), nh, nkv, hd, scale, window, **kw, **more)
    return out.cpu()


ATT_SHAPES = [  # heads, kv heads, head size, page size
    (4, 2, 16, 16), (3, 1, 32, 8), (6, 3, 48, 4), (8, 8, 64, 16), (8, 2, 128, 16), (5, 1, 80, 32),
    (20, 1, 16, 16)]
MIXED = [(700, 1), (129, 129), (64, 2), (333, 40), (1, 1), (65, 65), (200, 1)]
DECODE_FIRST = [(700, 1), (300, 1), (1, 1), (1500, 1), (129, 129), (64, 2), (333, 40), (77, 1), (65, 65)]
DECODE = [(700, 1), (129, 1), (64, 1), (1, 1), (65, 1), (1500, 1)]


@pytest.mark.parametrize("nh,nkv,hd,P", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
def test_attention_float32(ops, nh, nkv, hd, P, window):
    seqs = MIXED[:5]
    case = paged_case(seqs, nh, nkv, hd, P, torch.float32, seed=hd + P)
    scale = 1.0 / math.sqrt(hd)
    got = run_attention(ops, case, nh, nkv, hd, scale, window, tensor_cores=False)
    ref = reference_attention(case, seqs, nh, hd, window or None)
    assert rel_err(got, ref) < 2e-5


@pytest.mark.parametrize("nh,nkv,hd,P", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 37, 200])
@pytest.mark.parametrize("mode", ["mixed", "decode_first", "decode", "rows"])
def test_attention_bfloat16(ops, nh, nkv, hd, P, window, mode):
    seqs = DECODE if mode == "decode" else DECODE_FIRST if mode == "decode_first" else MIXED
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=hd + P + 1)
    scale = 0.7 / math.sqrt(hd)
    got = run_attention(ops, case, nh, nkv, hd, scale, window, tensor_cores=(mode != "rows"))
    ref = reference_attention(case, seqs, nh, hd, window or None, scale=scale)
    assert rel_err(got, ref) < 1.5e-2


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, False),
                                                (torch.bfloat16, True)])
@pytest.mark.parametrize("far", [0, 3, 15, 16, 63, 64, 127, 128, 500, 1023])
def test_attention_finds_one_far_key(ops, dtype, tensor_cores, far):
    """One key among a thousand is made to win the softmax; its value must come out.  A key
    that a kernel skips (a page's edge, a tile's edge, the first or last key) shows at once."""
    nh, nkv, hd, P = 4, 2, 32, 16
    ctx = 1024
    for seqs in ([(ctx, 1)], [(ctx, 5)]):
        case = paged_case(seqs, nh, nkv, hd, P, dtype, seed=far)
        k, v = case["ks"][0], case["vs"][0]
        qrow = case["rows_q"][0][-1]                       # the last row sees every key
        for h in range(nkv):
            k[far, h] = (qrow[h * 2].float() * 40.0 / qrow[h * 2].float().norm()).to(dtype)
            v[far, h] = torch.full((hd,), 3.0 + h).to(dtype)
        page = int(case["table"][0, far // P])
        case["cache"][page, 0, :, far % P] = k[far]
        case["cache"][page, 1, :, far % P] = v[far]
        # make the query long enough that the chosen key dominates
        for h in range(nkv):
            case["rows_q"][0][-1, h * 2] = (qrow[h * 2].float() * 3.0).to(dtype)
        case["q"] = torch.cat(case["rows_q"]).reshape(-1, nh * hd)
        got = run_attention(ops, case, nh, nkv, hd, 1.0, 0, tensor_cores).view(-1, nh, hd)[-1]
        ref = reference_attention(case, seqs, nh, hd, None, scale=1.0).view(-1, nh, hd)[-1]
        for h in range(nkv):
            assert abs(float(ref[h * 2].mean()) - (3.0 + h)) < 0.05       # the construction works
            assert float((got[h * 2].double() - ref[h * 2]).abs().max()) < (1e-4 if dtype == torch.float32 else 0.05)


@pytest.mark.parametrize("tensor_cores", [False, True])
def test_attention_window_edge_and_freed_pages(ops, tensor_cores):
    """Keys just inside and just outside the window, with the pages before the window given
    back (their table entries are -1 and must never be read)."""
    nh, nkv, hd, P, window = 2, 1, 16, 8, 20
    seqs = [(100, 1), (61, 3)]
    # the first visible key of a sequence's first query row is pos - window + 1
    freed = [100 - 1 - window + 1, 61 - 3 - window + 1]
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=3, freed_before=freed)
    for s, (ctx, qn) in enumerate(seqs):
        inside, outside = ctx - window, ctx - window - 1
        for pos, val in ((inside, 5.0), (outside, -7.0)):
            case["ks"][s][pos, 0] = (case["rows_q"][s][-1, 0].float() * 30 /
                                     case["rows_q"][s][-1, 0].float().norm()).bfloat16()
            case["vs"][s][pos, 0] = val
            page = int(case["table"][s, pos // P])
            if page >= 0:
                case["cache"][page, 0, :, pos % P] = case["ks"][s][pos]
                case["cache"][page, 1, :, pos % P] = case["vs"][s][pos]
    got = run_attention(ops, case, nh, nkv, hd, 1.0, window, tensor_cores)
    ref = reference_attention(case, seqs, nh, hd, window, scale=1.0)
    assert rel_err(got, ref) < 1.5e-2
    assert float(ref.view(-1, nh, hd)[0, 0].mean()) > 4.0     # the key at the window's edge is seen
