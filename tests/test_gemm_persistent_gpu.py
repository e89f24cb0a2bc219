"""The persistent tensor-core product against a plain 32-bit product: sizes that are no
multiple of a tile, fewer tiles than SMs and many more, and the fused gated activation over
alternating gate and up rows."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from allpaca_b200 import ops as o
    return o


# the last three: whole rounds of tiles and a rest that is shared out along K (88 tiles of 384, 12 of 160),
# and a rest of one tile
SHAPES = [(65, 128, 64), (128, 384, 256), (200, 1000, 520), (257, 4096, 1024), (700, 18944, 128), (2048, 1536, 4096),
          (2048, 6144, 512), (1100, 4000, 1024), (1000, 4800, 2048)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("share", [True, False])
def test_plain_product(ops, M, N, K, out_dtype, share):
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.5).bfloat16()
    out = torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)
    ops.gemm_tc_persistent(a.cuda(), w.cuda(), out, share_tiles=share)
    ops.check_kernel_status()
    ref = a.double() @ w.double().T
    tol = 1e-5 if out_dtype == torch.float32 else 5e-3
    assert float((out.cpu().double() - ref).abs().max() / ref.abs().max()) < tol


@pytest.mark.parametrize("M,I,K", [(65, 64, 64), (130, 333, 256), (513, 1409, 512), (2048, 2048, 1024), (600, 3000, 2048),
                                   (2048, 3072, 1024)])
def test_gated_activation_over_alternating_rows(ops, M, I, K):
    g = torch.Generator().manual_seed(M + I + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    gate = (torch.randn(I, K, generator=g) * 0.3).bfloat16()
    up = (torch.randn(I, K, generator=g) * 0.3).bfloat16()
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc_persistent(a.cuda(), w.cuda(), out, pairs=True)
    ops.check_kernel_status()
    gv = (a.double() @ gate.double().T).float().bfloat16().double()
    uv = (a.double() @ up.double().T).float().bfloat16().double()
    ref = gv / (1.0 + torch.exp(-gv)) * uv
    assert torch.isfinite(out).all()
    assert float((out.cpu().double() - ref).abs().max() / ref.abs().max()) < 1e-2


def test_shared_tiles_repeat_bit_for_bit_and_agree_with_whole_tiles(ops):
    """Few tiles, much K: every tile is shared by several CTAs that hand partial sums over.
    The flags must be left ready for the next product, the sums must not depend on timing, and
    the result must agree with whole tiles."""
    g = torch.Generator().manual_seed(3)
    for M, N, K, pairs in ((300, 2176, 4160, False), (576, 2048, 8192, False), (130, 512, 2048, True),
                           (2048, 6144, 1024, False), (1100, 4000, 1024, True), (256, 6144, 4096, False)):
        a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().cuda()
        w = (torch.randn(N, K, generator=g) * 0.5).bfloat16().cuda()
        n_out = N // 2 if pairs else N
        outs = []
        for _ in range(3):
            out = torch.full((M, n_out), float("nan"), device="cuda", dtype=torch.float32)
            ops.gemm_tc_persistent(a, w, out, pairs=pairs)
            outs.append(out)
        ops.check_kernel_status()
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        whole = torch.empty_like(outs[0])
        ops.gemm_tc_persistent(a, w, whole, pairs=pairs, share_tiles=False)
        scale = float(whole.abs().max())
        assert torch.isfinite(outs[0]).all()
        assert float((outs[0] - whole).abs().max()) / scale < (2e-2 if pairs else 1e-5)


def test_a_view_with_a_leading_dimension_is_refused_or_right(ops):
    """Shapes the kernel cannot take are refused with a message, never computed wrongly."""
    a = torch.randn(70, 60, device="cuda").bfloat16()          # K = 60: rows of 120 bytes
    w = torch.randn(128, 60, device="cuda").bfloat16()
    out = torch.empty(70, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(Exception, match="multiples of 8"):
        ops.gemm_tc_persistent(a, w, out)
