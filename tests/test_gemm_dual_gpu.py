"""The tensor-core product with two weight tiles per CTA, plain and with the gated
activation in its epilogue."""
import pytest
import torch

import plain_llama

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


@pytest.mark.parametrize("M,I,K", [(65, 176, 64), (100, 200, 120), (128, 256, 96), (300, 301 * 0 + 304, 1000),
                                   (513, 1000, 256), (2048, 896, 512)])
def test_dual_gated_activation(M, I, K):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(I)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, generator=g) * 0.1).bfloat16()
    out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc_dual(a.cuda(), w.cuda(), out, swiglu=True)
    ops.check_kernel_status()
    gate = (a.float() @ w[:I].float().T).bfloat16().float()
    up = (a.float() @ w[I:].float().T).bfloat16().float()
    ref = (plain_llama.silu(gate) * up).double()
    assert rel_err(out, ref) < 1e-2
