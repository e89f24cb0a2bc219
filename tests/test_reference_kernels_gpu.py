"""The reference's own CUDA kernels, compiled unchanged (``baseline/reference_kernels.py``), as
an oracle that is not this repository's reading of the formulas: each of them against the
plain implementation and against this engine's 32-bit kernel of the same operation, at the
tiny configurations' sizes and a few hundred keys.

The reference's kernels are 32-bit float throughout; its attention takes contiguous keys and
values, so the engine's paged cache is filled from the same tensors."""
import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

TOL = 1e-5          # of the largest element, against float64; both sides are 32-bit kernels


@pytest.fixture(scope="module")
def ref():
    from baseline import reference_kernels
    lib = reference_kernels.load()
    if lib is None:
        pytest.skip("the reference's kernels are not built here (no source tree beside the repository, or no nvcc)")
    return lib


@pytest.fixture(scope="module")
def ops():
    from allpaca_b200 import ops as o
    return o


def rel_err(got, want):
    want = want.double().cpu()
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).cuda()


@pytest.mark.parametrize("M,N,K", [(5, 176, 64), (31, 96, 256), (1, 301, 120), (40, 512, 96)])
def test_matrix_product(ref, ops, M, N, K):
    a, w = rand(M, K, seed=M), rand(N, K, seed=N, scale=0.05)
    theirs = torch.empty(M, N, device="cuda")
    ours = torch.empty(M, N, device="cuda")
    ref.gemm_nt(a, w, theirs)
    ops.gemm_simt(a, w, ours)
    want = a.double().cpu() @ w.double().cpu().T
    assert rel_err(theirs, want) < TOL and rel_err(ours, want) < TOL
    assert rel_err(ours, theirs) < TOL


@pytest.mark.parametrize("rows,H,eps", [(5, 64, 1e-5), (17, 96, 1e-6), (3, 120, 3e-6), (2, 4096, 1e-5)])
def test_rmsnorm(ref, ops, rows, H, eps):
    x, w = rand(rows, H, seed=H, scale=3.0), 1 + rand(H, seed=rows, scale=0.1)
    theirs = torch.empty_like(x)
    ours = torch.empty_like(x)
    ref.rmsnorm_rows(x, w, theirs, eps)
    ops.add_rmsnorm(x.clone(), w, eps, ours)
    want = plain_llama.rmsnorm(x.double().cpu(), w.double().cpu(), eps)
    assert rel_err(theirs, want) < TOL and rel_err(ours, want) < TOL and rel_err(ours, theirs) < TOL


def test_gated_activation_and_residual(ref, ops):
    T, inter = 7, 176
    gate, up = rand(T, inter, seed=1, scale=2.0), rand(T, inter, seed=2)
    theirs = torch.empty_like(gate)
    ref.silu_mul(gate, up, theirs)
    ours = torch.empty_like(gate)
    ops.swiglu(torch.cat([gate, up], dim=1).contiguous(), ours)
    want = plain_llama.silu(gate.double().cpu()) * up.double().cpu()
    assert rel_err(theirs, want) < TOL and rel_err(ours, want) < TOL and rel_err(ours, theirs) < TOL
    x, y = rand(T, 64, seed=3), rand(T, 64, seed=4)
    out = torch.empty_like(x)
    ref.residual_add(x, y, out)
    mine = x.clone()
    ops.residual_add(mine, y[None].contiguous())
    assert torch.equal(out, mine)


def test_embedding_row(ref, ops):
    table = rand(301, 120, seed=5)
    out = torch.empty(120, device="cuda")
    ref.embed_gather(table, 299, out)
    mine = torch.empty(1, 120, device="cuda")
    ops.embed_gather(torch.tensor([299], dtype=torch.int32, device="cuda"), table, mine)
    assert torch.equal(out, table[299]) and torch.equal(mine[0], out)


@pytest.mark.parametrize("pairing", ["adjacent", "half"])
@pytest.mark.parametrize("nh,nkv,hd,theta,start", [(4, 2, 16, 10000.0, 0), (3, 1, 32, 500000.0, 37),
                                                   (6, 3, 48, 25000.0, 5)])
def test_rotation(ref, ops, pairing, nh, nkv, hd, theta, start):
    """Both pairings the reference has: neighbours ``(2i, 2i+1)`` for checkpoints whose rows a
    converter permuted, ``(i, i + hd/2)`` for the Hugging Face layout.  The plain implementation's
    half-split rotation is the one the whole-model oracle uses."""
    T = 9
    q, k = rand(T, nh, hd, seed=hd), rand(T, nkv, hd, seed=hd + 1)
    tq, tk = q.clone(), k.clone()
    (ref.rope_adjacent if pairing == "adjacent" else ref.rope_half_split)(tq, tk, start, theta)
    positions = torch.arange(start, start + T)
    inv = plain_llama.rope_inverse_frequencies(hd, theta, None)

    def plain(x):
        x = x.double().cpu()
        if pairing == "half":
            return plain_llama.rope_half_split(x, positions, inv)
        # neighbours: bring (2i, 2i+1) to (i, i + half), rotate, and back
        split = torch.cat([x[..., 0::2], x[..., 1::2]], dim=-1)
        r = plain_llama.rope_half_split(split, positions, inv)
        out = torch.empty_like(r)
        out[..., 0::2], out[..., 1::2] = r[..., :hd // 2], r[..., hd // 2:]
        return out
    # angles are 32-bit products of up to ~45 with a frequency: a few 1e-6 of rounding in the angle
    assert rel_err(tq, plain(q)) < 5e-5 and rel_err(tk, plain(k)) < 5e-5
    # this engine's rotation (table of cos/sin, then rotate; no cache)
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), torch.zeros(T, nkv * hd, device="cuda")], dim=1).contiguous()
    table = torch.empty(T, hd // 2, 2, device="cuda")
    pos_dev = positions.to(torch.int32).cuda()
    ops.rope_table(pos_dev, inv.float().cuda(), table)
    q_out = torch.empty(T, nh * hd, device="cuda")
    ops.rope_kv_store(qkv, q_out, None, pos_dev, None, None, table, 1 if pairing == "adjacent" else 0, nh, nkv, hd)
    assert rel_err(q_out.view(T, nh, hd), tq) < 5e-5


@pytest.mark.parametrize("nh,nkv,hd,n_q,n_kv", [(4, 2, 16, 31, 31), (3, 1, 32, 1, 300), (6, 3, 48, 20, 150),
                                                (8, 2, 128, 5, 400), (4, 4, 64, 64, 64)])
def test_attention(ref, ops, nh, nkv, hd, n_q, n_kv):
    """Causal, grouped heads, the query rows being the last ``n_q`` positions of ``n_kv`` keys."""
    q = rand(n_q, nh, hd, seed=n_q)
    k, v = rand(n_kv, nkv, hd, seed=n_kv), rand(n_kv, nkv, hd, seed=n_kv + 1)
    # one key far back that a head must find: scale its match so that its score stands out
    k[3] = q[-1, ::nh // nkv] * 1.5
    theirs = torch.empty_like(q)
    ref.attention(q, k, v, theirs, causal=True)
    # the plain implementation takes whole sequences: give the earlier positions empty queries
    q_whole = torch.zeros(n_kv, nh, hd, dtype=torch.float64)
    q_whole[n_kv - n_q:] = q.double().cpu()
    want = plain_llama.causal_attention(q_whole, k.double().cpu(), v.double().cpu())[n_kv - n_q:]
    assert rel_err(theirs, want) < TOL
    # this engine's 32-bit attention over pages filled from the same keys and values
    P = 16
    pages = -(-n_kv // P)
    cache = torch.zeros(pages + 2, 2, nkv, P, hd, device="cuda")
    order = torch.randperm(pages + 2, generator=torch.Generator().manual_seed(1))[:pages]
    for i in range(pages):
        rows = slice(i * P, min((i + 1) * P, n_kv))
        n = rows.stop - rows.start
        cache[order[i], 0, :, :n] = k[rows].transpose(0, 1)
        cache[order[i], 1, :, :n] = v[rows].transpose(0, 1)
    table = order.to(torch.int32).cuda()[None].contiguous()
    positions = torch.arange(n_kv - n_q, n_kv, dtype=torch.int32, device="cuda")
    token_seq = torch.zeros(n_q, dtype=torch.int32, device="cuda")
    ours = torch.empty(n_q, nh * hd, device="cuda")
    ops.attention(q.reshape(n_q, -1).contiguous(), ours, cache, table, token_seq, positions, nh, nkv, hd,
                  hd ** -0.5)
    assert rel_err(ours.view(n_q, nh, hd), want) < TOL and rel_err(ours.view(n_q, nh, hd), theirs) < TOL
