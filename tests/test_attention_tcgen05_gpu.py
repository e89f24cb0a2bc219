"""The two tcgen05 attention kernels for prompt portions (one query tile to a CTA, and two:
``wide``) against the plain attention and against the mma.sync tile kernel: several
sequences, odd lengths, windows, pages given back, a far key that must be found."""
import math

import pytest
import torch

from test_kernels_gpu import paged_case, reference_attention, rel_err, run_attention

pytestmark = pytest.mark.gpu

SHAPES = [(8, 2, 128, 16), (32, 8, 128, 16), (4, 4, 128, 8), (16, 2, 64, 32), (8, 8, 64, 16), (16, 1, 128, 64)]
SEQS = [(700, 700), (129, 129), (333, 40), (64, 2), (257, 130), (1, 1), (200, 1)]
WIDE = pytest.mark.parametrize("wide", [False, True])


def supported(ops, nh, nkv, hd, P):
    from allpaca_b200.ops import library
    lib = library.attention(hd)
    return (hasattr(lib, "ap_attention_tcgen05") and bool(lib.ap_attention_tcgen05_supports(nh, nkv, hd, P))
            and bool(lib.ap_attention_tcgen05_wide_supports(nh, nkv, hd, P)))


@pytest.fixture(scope="module")
def ops():
    from allpaca_b200 import ops as o
    return o


@pytest.mark.parametrize("nh,nkv,hd,P", SHAPES)
@pytest.mark.parametrize("window", [0, 37, 300])
@pytest.mark.parametrize("sequential", [False, True])
@WIDE
def test_against_plain_and_tile_kernel(ops, nh, nkv, hd, P, window, sequential, wide):
    """Pages scattered over the pool (one load per page) and in rising order (one load per
    run of pages that fills a key tile)."""
    assert supported(ops, nh, nkv, hd, P)
    case = paged_case(SEQS, nh, nkv, hd, P, torch.bfloat16, seed=hd + P + window, sequential=sequential)
    scale = 0.9 / math.sqrt(hd)
    got = run_attention(ops, case, nh, nkv, hd, scale, window, tensor_cores=True, wide=wide)
    ops.check_kernel_status()
    ref = reference_attention(case, SEQS, nh, hd, window or None, scale=scale)
    assert rel_err(got, ref) < 1.5e-2
    # the mma.sync tile kernel on the same inputs
    q = case["q"].cuda()
    out = torch.empty_like(q)
    ops.attention(q, out, case["cache"].cuda(), case["table"].cuda(), case["token_seq"].cuda(),
                  case["positions"].cuda(), nh, nkv, hd, scale, window, seq_start=case["seq_start"].cuda(),
                  query_lens=case["query_lens"], max_context=int(case["positions"].max()) + 1, use_tcgen05=False)
    assert rel_err(out.cpu(), ref) < 1.5e-2
    assert rel_err(got, out.cpu().double()) < 1.5e-2


def test_unsupported_shapes_fall_back(ops):
    assert not supported(ops, 6, 2, 48, 16)          # head size 48
    assert not supported(ops, 6, 2, 128, 16)         # group 3 does not divide 128
    assert not supported(ops, 8, 2, 128, 4)          # page of 4
    assert not supported(ops, 8, 2, 128, 48)         # page that does not divide 128
    seqs = [(90, 90)]
    case = paged_case(seqs, 6, 2, 128, 16, torch.bfloat16, seed=1)
    got = run_attention(ops, case, 6, 2, 128, 0.1, 0, tensor_cores=True)
    assert rel_err(got, reference_attention(case, seqs, 6, 128, None, scale=0.1)) < 1.5e-2


@pytest.mark.parametrize("far", [0, 15, 16, 127, 128, 129, 255, 256, 600, 1023])
@WIDE
def test_finds_one_far_key(ops, far, wide):
    nh, nkv, hd, P = 4, 2, 64, 16
    ctx = 1024
    seqs = [(ctx, 70)]
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=far)
    k, v = case["ks"][0], case["vs"][0]
    qrow = case["rows_q"][0][-1]
    for h in range(nkv):
        k[far, h] = (qrow[h * 2].float() * 40.0 / qrow[h * 2].float().norm()).bfloat16()
        v[far, h] = torch.full((hd,), 3.0 + h).bfloat16()
    page = int(case["table"][0, far // P])
    case["cache"][page, 0, :, far % P] = k[far]
    case["cache"][page, 1, :, far % P] = v[far]
    for h in range(nkv):
        case["rows_q"][0][-1, h * 2] = (qrow[h * 2].float() * 3.0).bfloat16()
    case["q"] = torch.cat(case["rows_q"]).reshape(-1, nh * hd)
    got = run_attention(ops, case, nh, nkv, hd, 1.0, 0, tensor_cores=True, wide=wide).view(-1, nh, hd)[-1]
    ref = reference_attention(case, seqs, nh, hd, None, scale=1.0).view(-1, nh, hd)[-1]
    for h in range(nkv):
        assert abs(float(ref[h * 2].mean()) - (3.0 + h)) < 0.05
        assert float((got[h * 2].double() - ref[h * 2]).abs().max()) < 0.05


@pytest.mark.parametrize("sequential", [False, True])
@WIDE
def test_pages_given_back_are_not_read(ops, sequential, wide):
    nh, nkv, hd, P, window = 8, 2, 128, 16, 150
    seqs = [(900, 80), (500, 200)]
    freed = [900 - 80 - window + 1, 500 - 200 - window + 1]
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=9, freed_before=freed, sequential=sequential)
    got = run_attention(ops, case, nh, nkv, hd, 0.08, window, tensor_cores=True, wide=wide)
    ops.check_kernel_status()
    assert rel_err(got, reference_attention(case, seqs, nh, hd, window, scale=0.08)) < 1.5e-2


@pytest.mark.parametrize("rising", [True, False])
@WIDE
def test_scores_that_rise_or_fall_along_the_sequence(ops, rising, wide):
    """Rising scores move every row's reference maximum in every key tile, so the accumulator
    in tensor memory is scaled down again and again; falling scores never move it after the
    first tile, and the late probabilities are tiny."""
    nh, nkv, hd, P = 8, 2, 128, 16
    ctx = 1024
    seqs = [(ctx, ctx)]
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=5)
    g = torch.Generator().manual_seed(11)
    u = torch.randn(hd, generator=g)
    u = u / u.norm()
    ramp = torch.arange(ctx, dtype=torch.float32) / ctx
    if not rising:
        ramp = 1.0 - ramp
    k = case["ks"][0].float() * 0.1 + 14.0 * ramp[:, None, None] * u
    case["ks"][0] = k.bfloat16()
    case["rows_q"][0] = (case["rows_q"][0].float() * 0.1 + 14.0 * u).bfloat16()
    for j in range(ctx):
        page = int(case["table"][0, j // P])
        case["cache"][page, 0, :, j % P] = case["ks"][0][j]
    case["q"] = torch.cat(case["rows_q"]).reshape(-1, nh * hd)
    got = run_attention(ops, case, nh, nkv, hd, 1.0, 0, tensor_cores=True, wide=wide)
    ops.check_kernel_status()
    ref = reference_attention(case, seqs, nh, hd, None, scale=1.0)
    assert rel_err(got, ref) < 1.5e-2


@pytest.mark.parametrize("nh,nkv,hd,P", [(32, 8, 128, 16), (16, 2, 64, 32)])
@WIDE
def test_decoding_sequences_beside_prompt_portions(ops, nh, nkv, hd, P, wide):
    """A mixed batch in the scheduler's order, one-row sequences first: they run on the split
    kernel, the portions on the tcgen05 kernel, over disjoint rows of the same tensors."""
    seqs = [(900, 1), (17, 1), (2048, 1), (1, 1), (640, 1), (700, 512), (300, 300), (129, 1)]
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=21)
    scale = 1.0 / math.sqrt(hd)
    got = run_attention(ops, case, nh, nkv, hd, scale, 0, tensor_cores=True, wide=wide)
    ops.check_kernel_status()
    ref = reference_attention(case, seqs, nh, hd, None, scale=scale)
    assert rel_err(got, ref) < 1.5e-2
    # row by row: a row the wrong kernel wrote, or none wrote, shows here
    per_row = (got.double() - ref).abs().amax(dim=1) / ref.abs().max()
    assert float(per_row.max()) < 1.5e-2
