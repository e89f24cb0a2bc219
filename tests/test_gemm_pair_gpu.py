"""The tensor-core product on pairs of SMs (two CTAs to a tile of 256 weight rows x up to 256
tokens, ``tcgen05.mma.cta_group::2``), plain and with the gated activation in its epilogue."""
import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu


def rel_err(got, ref):
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


SHAPES = [(256, 256, 64), (65, 128, 512), (300, 520, 1032), (129, 384, 1024), (1000, 384, 2048), (2048, 1024, 512),
          (257, 4096, 4096), (700, 1000, 320), (2048, 6144, 4096),
          # few tiles of a long K: every tile is shared by two to four pairs, which hand partial sums over
          (512, 4096, 14336), (300, 1024, 8192), (200, 520, 6400),
          # more tiles than pairs, the last round of them partly filled (6 of 80, 21 of 95)
          (2048, 2560, 2048), (1100, 4864, 3072)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_pair_plain(M, N, K, odtype):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).bfloat16()
    out = torch.full((M + 2, N), 7.0, dtype=odtype, device="cuda")
    ops.gemm_tc_pair(a.cuda(), w.cuda(), out[:M])
    ops.check_kernel_status()
    ref = a.double() @ w.double().T
    assert rel_err(out[:M], ref) < (1e-5 if odtype == torch.float32 else 5e-3)
    assert torch.all(out[M:] == 7.0)
    again = torch.empty(M, N, dtype=odtype, device="cuda")
    ops.gemm_tc_pair(a.cuda(), w.cuda(), again)
    assert torch.equal(again, out[:M])


@pytest.mark.parametrize("M,I,K", [(65, 176, 64), (256, 128, 96), (300, 304, 1000), (513, 1000, 256), (2048, 896, 512),
                                   (300, 512, 4096), (140, 200, 9000 // 8 * 8), (2048, 1280, 2048)])
def test_pair_gated_activation(M, I, K):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(I)
    a = torch.randn(M, K, generator=g).bfloat16()
    gate = (torch.randn(I, K, generator=g) * 0.1).bfloat16()
    up = (torch.randn(I, K, generator=g) * 0.1).bfloat16()
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc_pair(a.cuda(), w.cuda(), out, pairs=True)
    ops.check_kernel_status()
    gv = (a.double() @ gate.double().T).float().bfloat16().double()
    uv = (a.double() @ up.double().T).float().bfloat16().double()
    ref = plain_llama.silu(gv) * uv
    assert torch.isfinite(out).all()
    assert rel_err(out, ref) < 1e-2


def test_shared_tiles_agree_with_whole_tiles_and_leave_the_flags_ready():
    """The same product with every tile's K shared among several pairs and with whole tiles: equal up
    to the order of the additions, and the same bits every time (the flags the pairs raise for one
    another are left ready for the next product)."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(9)
    for M, N, K in ((512, 4096, 14336), (300, 1024, 8192), (200, 520, 6400)):
        a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().cuda()
        w = (torch.randn(N, K, generator=g) * 0.5).bfloat16().cuda()
        outs = []
        for _ in range(4):
            out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
            ops.gemm_tc_pair(a, w, out)
            outs.append(out)
        ops.check_kernel_status()
        assert all(torch.equal(outs[0], o) for o in outs[1:])
        whole = torch.empty_like(outs[0])
        ops.gemm_tc_pair(a, w, whole, share_tiles=False)
        # against the exact product: the shared sums within 1e-5; one 32-bit accumulator over all of a K
        # of 14336 is the less exact of the two (1.7e-5 seen), so it gets 3e-5
        ref = a.double().cpu() @ w.double().cpu().T
        assert rel_err(outs[0], ref) < 1e-5 and rel_err(whole, ref) < 3e-5
        assert not torch.equal(outs[0], whole)                   # the shared path was really taken
