"""The decode-attention entry point that allocates nothing (`ap_attention_decode_static`).

Some users of the kernel library cannot allocate device memory around a call: they run
inside a fixed carve-out of memory, or in a loop that may not touch the allocator.  For
them the library keeps the scratch of the split-key attention kernel in a fixed array of
its own.  This test calls that entry point through its exported C symbol, twice in a row
(the second call meets whatever the first left in the array), and checks both results
against the regular entry point, which takes its scratch from the caller, and against a
plain float64 attention over the same keys and values (so that the two entry points cannot
be wrong together).  It also checks that a call whose scratch would not fit is refused with
a message.

The file sorts last so that a run that stops at the first failure has already run
everything else; it passes alone in a fresh process as well.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

NH, NKV, HD, P = 8, 2, 64, 16


def _library():
    from allpaca_b200.csrc import build
    lib = ctypes.CDLL(build.build_attention(HD))
    c = ctypes
    lib.ap_attention_decode_static.argtypes = [
        c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_int, c.c_int,
        c.c_int, c.c_int, c.c_longlong, c.c_float, c.c_int, c.c_int, c.c_void_p]
    lib.ap_attention_decode_static.restype = c.c_int
    lib.ap_last_error.restype = c.c_char_p
    return lib


def _case(seed, contexts):
    g = torch.Generator().manual_seed(seed)
    T = len(contexts)
    max_pages = max(-(-c // P) for c in contexts)
    pages = sum(-(-c // P) for c in contexts) + 2
    cache = torch.randn(pages, 2, NKV, P, HD, generator=g).bfloat16().cuda()
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((T, max_pages), -1, dtype=torch.int32)
    for s, c in enumerate(contexts):
        for j in range(-(-c // P)):
            table[s, j] = order.pop()
    q = torch.randn(T, NH * HD, generator=g).bfloat16().cuda()
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32).cuda()
    return q, cache, table.cuda(), positions


def _regular(q, cache, table, positions, scale, window):
    from allpaca_b200 import ops
    T = q.shape[0]
    out = torch.empty_like(q)
    held = []

    def scratch(name, shape, dtype):
        held.append(torch.empty(shape, dtype=dtype, device="cuda"))
        return held[-1]
    ops.attention(q, out, cache, table, torch.arange(T, dtype=torch.int32, device="cuda"), positions,
                  NH, NKV, HD, scale, window,
                  seq_start=torch.arange(T + 1, dtype=torch.int32, device="cuda"),
                  query_lens=[1] * T, max_context=int(positions.max()) + 1, scratch=scratch)
    return out


def _plain(q, cache, table, positions, window):
    """Every sequence's single query row against its own keys, gathered page by page, with the
    plain implementation under tests/ (whole sequences: earlier positions get empty queries)."""
    import plain_llama
    out = torch.empty(q.shape[0], NH, HD, dtype=torch.float64)
    cache, table = cache.double().cpu(), table.cpu()
    for s in range(q.shape[0]):
        n = int(positions[s]) + 1
        pages = table[s, : -(-n // P)].long()
        k = cache[pages, 0].permute(0, 2, 1, 3).reshape(-1, NKV, HD)[:n]
        v = cache[pages, 1].permute(0, 2, 1, 3).reshape(-1, NKV, HD)[:n]
        whole = torch.zeros(n, NH, HD, dtype=torch.float64)
        whole[-1] = q[s].double().cpu().view(NH, HD)
        out[s] = plain_llama.causal_attention(whole, k, v, window=window or None)[-1]
    return out.view(q.shape[0], NH * HD)


def test_static_scratch_entry_matches_the_regular_one_twice():
    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(HD)
    for call, (seed, contexts, nsplit, window) in enumerate([(1, [700, 33, 1, 257, 64], 5, 0),
                                                             (2, [90, 1500, 16], 9, 300)]):
        q, cache, table, positions = _case(seed, contexts)
        want = _regular(q, cache, table, positions, scale, window)
        got = torch.empty_like(q)
        rc = lib.ap_attention_decode_static(
            q.data_ptr(), got.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1],
            positions.data_ptr(), q.shape[0], NH, NKV, HD, P, cache.stride(0), scale, window, nsplit, stream)
        assert rc == 0, lib.ap_last_error().decode()
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        # the same kernels with a different number of key slices: the tolerance of the
        # bfloat16 attention tests
        assert err < 1.5e-2, f"call {call}: error {err:.3e}"
        plain = _plain(q, cache, table, positions, window)
        for what, t in (("static scratch", got), ("regular", want)):
            err = float((t.double().cpu() - plain).abs().max() / plain.abs().max())
            assert err < 1.5e-2, f"call {call}: {what} entry is {err:.3e} off the plain attention"


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = _library()
    q, cache, table, positions = _case(3, [64] * 64)
    out = torch.empty_like(q)
    rc = lib.ap_attention_decode_static(
        q.data_ptr(), out.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1],
        positions.data_ptr(), q.shape[0], NH, NKV, HD, P, cache.stride(0), 0.125, 0, 100,
        torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.ap_last_error().decode()
    assert "scratch" in msg and "floats" in msg
    rc = lib.ap_attention_decode_static(
        q.data_ptr(), out.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1],
        positions.data_ptr(), q.shape[0], NH, NKV, 48, P, cache.stride(0), 0.125, 0, 1,
        torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "head size" in lib.ap_last_error().decode()
