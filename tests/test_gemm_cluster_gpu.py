"""The tensor-core matrix product with its K slices added inside a thread-block cluster."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_err(got, ref):
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


@pytest.mark.parametrize("M,N,K,S", [(1, 128, 512, 2), (8, 301, 1000, 3), (16, 256, 4096, 8), (8, 4096, 4096, 7),
                                     (64, 384, 1024, 4), (5, 640, 14336, 8), (33, 130, 640, 5), (17, 6144, 4096, 6)])
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_cluster_reduction(M, N, K, S, odtype):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(S + M)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).bfloat16()
    out = torch.full((M + 1, N), 7.0, dtype=odtype, device="cuda")
    ops.gemm_tc(a.cuda(), w.cuda(), out[:M], S, reduce=True)
    ops.check_kernel_status()
    ref = a.double() @ w.double().T
    assert rel_err(out[:M], ref) < (1e-5 if odtype == torch.float32 else 5e-3)
    assert torch.all(out[M:] == 7.0)
    # the same product twice gives the same bits: slices are added in a fixed order
    again = torch.empty(M, N, dtype=odtype, device="cuda")
    ops.gemm_tc(a.cuda(), w.cuda(), again, S, reduce=True)
    assert torch.equal(again, out[:M])


def test_plan_stays_within_a_cluster():
    from allpaca_b200 import ops
    for M in (1, 8, 16, 33, 64, 65, 128, 200, 256):
        for N, K in ((4096, 4096), (6144, 4096), (28672, 4096), (4096, 14336), (128256, 4096), (96, 64)):
            s = ops.gemm_tc_splits(M, N, K)
            kb = -(-K // 64)
            assert 1 <= s <= 8 and (s - 1) * (-(-kb // s)) < kb
            assert M <= 128 or s != 2         # tiles of 256 tokens: two slices do not pay: four or more, or none
    # up to 256 rows against few weight tiles are split (two CTAs to an SM up to 128 rows, one beyond); more rows never
    assert ops.gemm_tc_splits(64, 4096, 4096) == 8 and ops.gemm_tc_splits(128, 6144, 4096) == 4
    assert ops.gemm_tc_splits(129, 4096, 4096) == 4 and ops.gemm_tc_splits(257, 4096, 4096) == 1
    assert ops.gemm_tc_splits(2048, 4096, 4096) == 1 and ops.gemm_tc_splits(200, 28672, 4096) == 1


def test_cluster_reduction_refuses_too_many_slices():
    from allpaca_b200 import ops
    a = torch.randn(4, 4608).bfloat16().cuda()
    w = torch.randn(128, 4608).bfloat16().cuda()
    out = torch.empty(4, 128, device="cuda")
    with pytest.raises(ops.KernelError, match="cluster"):
        ops.gemm_tc(a, w, out, 9, reduce=True)


@pytest.mark.parametrize("M,I,K,nsplit", [(1, 64, 512, 1), (8, 200, 512, 4), (8, 1409, 1024, 8), (33, 96, 256, 2),
                                          (64, 300, 512, 1), (5, 7168, 256, 1)])
def test_gated_epilogue_over_alternating_rows(M, I, K, nsplit):
    """Few rows: silu(gate) * up straight from the product, gate and up rows alternating, with
    the K slices added in a cluster or none at all."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + I + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    gate = (torch.randn(I, K, generator=g) * 0.3).bfloat16()
    up = (torch.randn(I, K, generator=g) * 0.3).bfloat16()
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc(a.cuda(), w.cuda(), out, nsplit, reduce=nsplit > 1, pairs=True)
    ops.check_kernel_status()
    gv = (a.double() @ gate.double().T).float().bfloat16().double()
    uv = (a.double() @ up.double().T).float().bfloat16().double()
    ref = gv / (1.0 + torch.exp(-gv)) * uv
    assert torch.isfinite(out).all()
    assert float((out.cpu().double() - ref).abs().max() / ref.abs().max()) < 1e-2


@pytest.mark.parametrize("M,N,K,nsplit", [(65, 128, 512, 2), (128, 384, 1024, 4), (188, 520, 2048, 8), (256, 256, 4096, 4),
                                          (200, 1000, 1032, 2), (130, 4096, 4096, 4)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_cluster_reduction_with_up_to_256_rows(M, N, K, nsplit, out_dtype):
    """65 to 256 rows: the buffer the slices are gathered in lies over the operand stages."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.5).bfloat16()
    outs = []
    for _ in range(2):
        out = torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)
        ops.gemm_tc(a.cuda(), w.cuda(), out, nsplit, reduce=True)
        outs.append(out)
    ops.check_kernel_status()
    assert torch.equal(outs[0], outs[1])
    ref = a.double() @ w.double().T
    tol = 1e-5 if out_dtype == torch.float32 else 5e-3
    assert float((outs[0].cpu().double() - ref).abs().max() / ref.abs().max()) < tol


@pytest.mark.parametrize("M,I,K,nsplit", [(100, 200, 512, 2), (256, 1409, 1024, 4), (129, 64, 2048, 8)])
def test_gated_epilogue_with_up_to_256_rows(M, I, K, nsplit):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + I + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    gate = (torch.randn(I, K, generator=g) * 0.3).bfloat16()
    up = (torch.randn(I, K, generator=g) * 0.3).bfloat16()
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc(a.cuda(), w.cuda(), out, nsplit, reduce=True, pairs=True)
    ops.check_kernel_status()
    gv = (a.double() @ gate.double().T).float().bfloat16().double()
    uv = (a.double() @ up.double().T).float().bfloat16().double()
    ref = gv / (1.0 + torch.exp(-gv)) * uv
    assert torch.isfinite(out).all()
    assert float((out.cpu().double() - ref).abs().max() / ref.abs().max()) < 1e-2


@pytest.mark.parametrize("M,N,K,nsplit", [(1, 128, 512, 1), (8, 4096, 4096, 8), (8, 4096, 2048, 4), (33, 520, 1024, 2),
                                          (64, 384, 512, 1), (5, 4096, 14336, 8), (16, 304, 640, 4),
                                          (64, 2048, 8192, 8)])
def test_residual_epilogue(M, N, K, nsplit):
    """The product adds into the 32-bit residual itself, keeps a bfloat16 copy of the updated
    rows and sums their squares in parts; rows beyond M are not touched."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + N + nsplit)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    x0 = torch.randn(M + 1, N, generator=g) * 2
    x = x0.clone().cuda()
    xb = torch.full((M + 1, N), 3.0, dtype=torch.bfloat16, device="cuda")
    parts = ops.gemm_tc_residual_parts(N, nsplit)
    ss = torch.full((M + 1, parts), -1.0, device="cuda")
    got_parts = ops.gemm_tc_residual(a.cuda(), w.cuda(), x[:M], xb[:M], ss[:M], nsplit)
    ops.check_kernel_status()
    assert got_parts == parts
    ref = x0[:M].double() + a.double() @ w.double().T
    assert rel_err(x[:M], ref) < 1e-5
    assert torch.equal(x[M:].cpu(), x0[M:]) and torch.all(xb[M:] == 3.0) and torch.all(ss[M:] == -1.0)
    assert torch.equal(xb[:M], x[:M].bfloat16())                       # the copy is the rounding of what was stored
    assert (ss[:M] >= 0).all()                                         # every part was written
    want = (x[:M].double() ** 2).sum(1).cpu()
    assert float(((ss[:M].double().sum(1).cpu() - want).abs() / want).max()) < 1e-5
    # twice the same bits
    x2, xb2, ss2 = x0.clone().cuda(), torch.empty_like(xb), torch.empty_like(ss)
    ops.gemm_tc_residual(a.cuda(), w.cuda(), x2[:M], xb2[:M], ss2[:M], nsplit)
    assert torch.equal(x2[:M], x[:M]) and torch.equal(ss2[:M], ss[:M])


@pytest.mark.parametrize("M,N,K,nsplit", [(1, 128, 512, 1), (8, 6144, 4096, 4), (33, 520, 1024, 2), (64, 384, 512, 1),
                                          (7, 1000, 2048, 8)])
@pytest.mark.parametrize("pairs", [False, True])
def test_rows_scaled_by_a_deferred_norm(M, N, K, nsplit, pairs):
    """The product's result rows multiplied by 1/sqrt(mean square + eps) of its input rows, the
    mean square given as partial sums: an RMSNorm applied after the product."""
    import plain_llama
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    parts, width, eps = 13, 777, 1e-3
    ss = torch.rand(M, parts, generator=g) * 50
    scale = ops.RowScale(ss.cuda(), parts, width, eps)
    inv = 1.0 / torch.sqrt(ss.double().sum(1) / width + eps)
    full = (a.double() @ w.double().T) * inv[:, None]
    if pairs:
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
        ops.gemm_tc(a.cuda(), w.cuda(), out, nsplit, reduce=nsplit > 1, pairs=True, scale=scale)
        gate, up = full[:, 0::2].float().bfloat16().double(), full[:, 1::2].float().bfloat16().double()
        ref = plain_llama.silu(gate) * up
        tol = 2e-2
    else:
        out = torch.empty(M, N, dtype=torch.float32, device="cuda")
        ops.gemm_tc(a.cuda(), w.cuda(), out, nsplit, reduce=nsplit > 1, scale=scale)
        ref, tol = full, 1e-5
    ops.check_kernel_status()
    assert rel_err(out, ref) < tol


@pytest.mark.parametrize("M,nh,nkv,hd,K,nsplit", [(1, 4, 2, 64, 256, 1), (8, 32, 8, 128, 4096, 4), (40, 3, 1, 32, 512, 2),
                                                  (64, 6, 3, 48, 384, 1), (7, 8, 2, 128, 1024, 8)])
@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("scaled", [False, True])
def test_rotation_and_cache_store_in_the_projection(M, nh, nkv, hd, K, nsplit, pairing, scaled):
    """The stacked Q, K, V projection with the rotation of Q and K and the store of K and V into
    pages in its epilogue, against the plain projection, rotation and placement.  For the
    half-split pairing the rows of each Q and K head are interleaved first, as the attention
    part does at load."""
    import plain_llama
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + nh + hd + K)
    P = 16
    a = torch.randn(M, K, generator=g).bfloat16()
    wq, wk, wv = (torch.randn(n * hd, K, generator=g).mul(0.05).bfloat16() for n in (nh, nkv, nkv))
    positions = torch.randint(0, 5 * P, (M,), generator=g).to(torch.int32)
    token_seq = torch.arange(M, dtype=torch.int32)
    table = torch.randperm(M * 5, generator=g).to(torch.int32).view(M, 5)
    inv = plain_llama.rope_inverse_frequencies(hd, 10000.0, None)
    parts, width, eps = 7, K, 1e-5
    ss = torch.rand(M, parts, generator=g) * 30
    row_scale = (1.0 / torch.sqrt(ss.double().sum(1) / width + eps)) if scaled else torch.ones(M, dtype=torch.float64)

    def proj(w, heads):
        return ((a.double() @ w.double().T) * row_scale[:, None]).float().bfloat16().double().view(M, heads, hd)
    q, k, v = proj(wq, nh), proj(wk, nkv), proj(wv, nkv)
    if pairing == 0:
        qr, kr = plain_llama.rope_half_split(q, positions, inv), plain_llama.rope_half_split(k, positions, inv)
        order = torch.stack([torch.arange(hd // 2), torch.arange(hd // 2) + hd // 2], dim=1).reshape(-1)
        wq_in = wq.view(nh, hd, K)[:, order].reshape(nh * hd, K)
        wk_in = wk.view(nkv, hd, K)[:, order].reshape(nkv * hd, K)
    else:
        def adjacent(x):
            split = torch.cat([x[..., 0::2], x[..., 1::2]], dim=-1)
            r = plain_llama.rope_half_split(split, positions, inv)
            out = torch.empty_like(r)
            out[..., 0::2], out[..., 1::2] = r[..., :hd // 2], r[..., hd // 2:]
            return out
        qr, kr = adjacent(q), adjacent(k)
        wq_in, wk_in = wq, wk
    w = torch.cat([wq_in, wk_in, wv]).contiguous().cuda()
    cos_sin = torch.empty(M, hd // 2, 2, device="cuda")
    ops.rope_table(positions.cuda(), inv.float().cuda(), cos_sin)
    q_out = torch.empty(M, nh * hd, dtype=torch.bfloat16, device="cuda")
    cache = torch.full((M * 5, 2, nkv, P, hd), 9.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc_rope(a.cuda(), w, q_out, cache, positions.cuda(), token_seq.cuda(), table.cuda(), cos_sin, pairing,
                     nh, nkv, hd, nsplit, ops.RowScale(ss.cuda(), parts, width, eps) if scaled else None)
    ops.check_kernel_status()
    tol = 1.2e-2
    assert rel_err(q_out.view(M, nh, hd), qr) < tol
    got = cache.cpu()
    touched = torch.zeros(M * 5, P, dtype=torch.bool)
    for t in range(M):
        page, slot = int(table[t, int(positions[t]) // P]), int(positions[t]) % P
        touched[page, slot] = True
        assert rel_err(got[page, 0, :, slot], kr[t]) < tol and rel_err(got[page, 1, :, slot], v[t]) < tol
    assert torch.all(got.permute(0, 3, 1, 2, 4)[~touched] == 9.0)           # nothing else was written
    # and without a cache only the queries are produced
    q2 = torch.empty_like(q_out)
    ops.gemm_tc_rope(a.cuda(), w, q2, None, positions.cuda(), None, None, cos_sin, pairing, nh, nkv, hd, nsplit,
                     ops.RowScale(ss.cuda(), parts, width, eps) if scaled else None)
    assert torch.equal(q2, q_out)
