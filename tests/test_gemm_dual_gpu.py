"""The tensor-core product with two weight tiles per CTA."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_err(got, ref):
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


SHAPES = [(65, 256, 64), (100, 257, 72), (128, 512, 136), (129, 384, 1024), (200, 128, 64), (256, 1000, 320),
          (300, 640, 1000), (700, 384, 2048), (2048, 1024, 512)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_dual_plain(M, N, K, odtype):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g).bfloat16()
    out = torch.full((M + 2, N), 7.0, dtype=odtype, device="cuda")
    ops.gemm_tc_dual(a.cuda(), w.cuda(), out[:M])
    ops.check_kernel_status()
    assert rel_err(out[:M], a.double() @ w.double().T) < (1e-5 if odtype == torch.float32 else 5e-3)
    assert torch.all(out[M:] == 7.0)
