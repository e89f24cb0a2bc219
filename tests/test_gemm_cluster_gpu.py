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
            assert M <= 64 or s != 2          # from 65 rows on two slices do not pay: four or more, or none
    # 65 to 256 rows against few weight tiles are still split; more rows never
    assert ops.gemm_tc_splits(65, 4096, 4096) == 4 and ops.gemm_tc_splits(257, 4096, 4096) == 1
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
