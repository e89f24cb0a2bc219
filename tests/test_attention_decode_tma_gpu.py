"""The TMA-fed decode attention kernel against the plain attention and the cp.async kernel:
page sizes, groups, windows, pages given back, forced numbers of key slices, and a far key
that must be found wherever it lies in a tile or a page."""
import math

import pytest
import torch

from test_kernels_gpu import dev, paged_case, reference_attention, rel_err

pytestmark = pytest.mark.gpu

SHAPES = [(8, 2, 128, 16), (32, 8, 128, 16), (4, 4, 128, 8), (16, 2, 64, 32), (8, 8, 64, 16), (16, 1, 128, 64),
          (40, 2, 64, 16), (32, 8, 128, 128), (8, 2, 64, 256), (8, 8, 64, 128)]
DECODE = [(700, 1), (129, 1), (64, 1), (1, 1), (65, 1), (1500, 1), (3000, 1)]


@pytest.fixture(scope="module")
def ops():
    from allpaca_b200 import ops as o
    return o


def run(ops, case, nh, nkv, hd, scale, window, use_tma, splits=None, monkeypatch=None):
    q = dev(case["q"])
    out = torch.full_like(q, float("nan"))
    keep = []

    def scratch(name, shape, dtype):
        keep.append(torch.empty(shape, dtype=dtype, device="cuda"))
        return keep[-1]
    if splits is not None:
        monkeypatch.setattr(ops, "decode_splits", lambda *a, **k: splits)
    ops.attention(q, out, dev(case["cache"]), dev(case["table"]), dev(case["token_seq"]), dev(case["positions"]),
                  nh, nkv, hd, scale, window, seq_start=dev(case["seq_start"]), query_lens=case["query_lens"],
                  max_context=int(case["positions"].max()) + 1, scratch=scratch, use_tma=use_tma)
    ops.check_kernel_status()
    return out.cpu()


def test_shapes_are_taken_or_left(ops):
    from allpaca_b200.ops import library
    lib = library.attention(128)
    assert lib.ap_attention_decode_tma_supports(32, 8, 128, 16)
    assert not lib.ap_attention_decode_tma_supports(32, 8, 128, 4)       # page of 4: below one swizzle atom
    assert not lib.ap_attention_decode_tma_supports(32, 8, 128, 48)      # does not divide a tile
    assert lib.ap_attention_decode_tma_supports(32, 8, 128, 128)         # two tiles to a page
    assert not lib.ap_attention_decode_tma_supports(32, 8, 128, 96)      # no whole number of tiles
    assert not lib.ap_attention_decode_tma_supports(32, 8, 64, 16)       # another head size's library
    assert not library.attention(48).ap_attention_decode_tma_supports(6, 2, 48, 16)


@pytest.mark.parametrize("nh,nkv,hd,P", SHAPES)
@pytest.mark.parametrize("window", [0, 37, 300])
@pytest.mark.parametrize("sequential", [False, True])
def test_against_plain_and_cp_async(ops, nh, nkv, hd, P, window, sequential):
    """Pages scattered over the pool (one load per page) and in rising order (one load per
    run of pages that fills a key tile)."""
    case = paged_case(DECODE, nh, nkv, hd, P, torch.bfloat16, seed=hd + P + window, sequential=sequential)
    scale = 0.9 / math.sqrt(hd)
    got = run(ops, case, nh, nkv, hd, scale, window, use_tma=True)
    ref = reference_attention(case, DECODE, nh, hd, window or None, scale=scale)
    assert rel_err(got, ref) < 1.5e-2
    other = run(ops, case, nh, nkv, hd, scale, window, use_tma=False)
    assert rel_err(got, other.double()) < 1.5e-2


@pytest.mark.parametrize("splits", [1, 2, 3, 4, 7, 8, 16, 24, 47])
@pytest.mark.parametrize("nh,nkv,hd,P", [(8, 2, 128, 16), (16, 1, 128, 64), (40, 2, 64, 16), (8, 2, 128, 128)])
def test_any_number_of_key_slices(ops, splits, nh, nkv, hd, P, monkeypatch):
    """Slices that hold one tile, many tiles or none at all (more slices than tiles); 2, 4, 8
    and 16 slices are combined inside a thread-block cluster where their results fit, the other
    counts by a second kernel."""
    case = paged_case(DECODE, nh, nkv, hd, P, torch.bfloat16, seed=splits)
    got = run(ops, case, nh, nkv, hd, 0.08, 0, use_tma=True, splits=splits, monkeypatch=monkeypatch)
    ref = reference_attention(case, DECODE, nh, hd, None, scale=0.08)
    assert rel_err(got, ref) < 1.5e-2


@pytest.mark.parametrize("far", [0, 7, 8, 15, 16, 63, 64, 127, 128, 500, 1023])
@pytest.mark.parametrize("P", [16, 128])
def test_finds_one_far_key(ops, far, P):
    nh, nkv, hd = 4, 2, 64
    ctx = 1024
    seqs = [(ctx, 1), (ctx - 3, 1)]
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
    got = run(ops, case, nh, nkv, hd, 1.0, 0, use_tma=True).view(-1, nh, hd)[0]
    ref = reference_attention(case, seqs, nh, hd, None, scale=1.0).view(-1, nh, hd)[0]
    for h in range(nkv):
        assert abs(float(ref[h * 2].mean()) - (3.0 + h)) < 0.05
        assert float((got[h * 2].double() - ref[h * 2]).abs().max()) < 0.05


@pytest.mark.parametrize("sequential", [False, True])
@pytest.mark.parametrize("P", [16, 128])
def test_pages_given_back_are_not_read(ops, sequential, P):
    nh, nkv, hd, window = 8, 2, 128, 150
    seqs = [(900, 1), (500, 1), (149, 1)]
    freed = [900 - 1 - window + 1, 500 - 1 - window + 1, 0]
    case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=9, freed_before=freed, sequential=sequential)
    got = run(ops, case, nh, nkv, hd, 0.08, window, use_tma=True)
    assert rel_err(got, reference_attention(case, seqs, nh, hd, window, scale=0.08)) < 1.5e-2
