"""Decode attention whose last key slice combines all slices itself (arrival counters in
zeroed scratch) against the variant with a separate combining kernel, over several launches
that reuse the same counters."""
import math

import pytest
import torch

from test_kernels_gpu import DECODE, paged_case, reference_attention, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nh,nkv,hd,P", [(8, 2, 128, 16), (3, 1, 32, 8), (20, 1, 16, 16), (6, 3, 48, 4)])
def test_last_slice_combines(nh, nkv, hd, P):
    from allpaca_b200 import ops
    zeroed, held = {}, []

    def scratch(name, shape, dtype):
        held.append(torch.empty(shape, dtype=dtype, device="cuda"))     # kept alive: the kernel owns it
        return held[-1]

    def zero_scratch(name, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        if name not in zeroed or zeroed[name].numel() < n:
            zeroed[name] = torch.zeros(n, dtype=dtype, device="cuda")
        return zeroed[name][:n].view(*shape)

    scale = 1.0 / math.sqrt(hd)
    for launch, window in enumerate([0, 0, 300, 0]):
        seqs = DECODE if launch % 2 == 0 else DECODE[::-1]
        case = paged_case(seqs, nh, nkv, hd, P, torch.bfloat16, seed=launch + hd)
        q = case["q"].cuda()
        outs = []
        for zs in (zero_scratch, None):
            out = torch.empty_like(q)
            ops.attention(q, out, case["cache"].cuda(), case["table"].cuda(), case["token_seq"].cuda(),
                          case["positions"].cuda(), nh, nkv, hd, scale, window,
                          seq_start=case["seq_start"].cuda(), query_lens=case["query_lens"],
                          max_context=int(case["positions"].max()) + 1, scratch=scratch, zero_scratch=zs)
            outs.append(out.cpu())
        ref = reference_attention(case, seqs, nh, hd, window or None, scale=scale)
        assert rel_err(outs[0], ref) < 1.5e-2 and rel_err(outs[1], ref) < 1.5e-2
        assert torch.equal(outs[0], outs[1])            # the same sums in the same order
        for buf in zeroed.values():
            assert int(buf.abs().sum()) == 0            # the counters are zero again
