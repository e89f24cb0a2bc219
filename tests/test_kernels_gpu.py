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
    ops.rope_kv_store(dev(inp), q_out, cd, dev(positions), dev(token_seq), dev(table),
                      dev(inv.float()), 0, nh, nkv, hd)
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
    ops.rope_kv_store(dev(x), out, None, dev(positions), None, None, dev(inv.float()), 1, nh, 0, hd)
    xv = x.double().view(T, nh, hd // 2, 2)
    ang = positions.double()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    ref = torch.stack([xv[..., 0] * c - xv[..., 1] * s, xv[..., 0] * s + xv[..., 1] * c], -1)
    assert rel_err(out.cpu().view(T, nh, hd // 2, 2), ref) < 2e-5
    ops.rope_kv_store(dev(x), out, None, dev(positions), None, None, None, 0, nh, 0, hd)
    assert torch.equal(out.cpu(), x)


# ---------------------------------------------------------------- gated activation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(ops, dtype):
    g = torch.Generator().manual_seed(2)
    T, I = 5, 177
    S = 3 if dtype == torch.float32 else 1
    gu = torch.randn(S, T, 2 * I, generator=g) * 2
    inp = gu if dtype == torch.float32 else gu[0].to(dtype)
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    ops.swiglu(dev(inp), out)
    full = (gu.sum(0) if dtype == torch.float32 else inp.float()).double()
    ref = plain_llama.silu(full[:, :I]) * full[:, I:]
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


@pytest.mark.parametrize("V", [64, 301, 5000])
def test_sample_matches_plain(ops, V):
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
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(torch.tensor([c[0] for c in cases])),
               dev(torch.tensor([c[1] for c in cases], dtype=torch.int32)),
               dev(torch.tensor([c[2] for c in cases])), dev(torch.tensor([c[3] for c in cases])), out)
    got = out.cpu().tolist()
    for r, (temp, k, p, u) in enumerate(cases):
        want = plain_llama.sample_plain(logits[r], temp, k, p, u)
        if got[r] != want:
            # allowed only when u sits on a boundary of the cumulative distribution (rounding)
            alt = {plain_llama.sample_plain(logits[r], temp, k, p, min(max(u + d, 0.0), 0.999999))
                   for d in (-2e-6, 2e-6)}
            assert got[r] in alt, (r, cases[r], got[r], want)


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
