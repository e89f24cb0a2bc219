"""The C++ step builder: what it writes for a mixed batch, what it refuses, and that a refused
step changes nothing (no GPU needed)."""
import numpy as np
import pytest

from allpaca_b200.cache import CacheManager, FREED, GroupLayout, OutOfPages
from allpaca_b200.engine.batch import BatchEntry
from allpaca_b200.engine.step_builder import StepError, build_step


def make(num_pages=16, page=4, max_seqs=3, window=None):
    groups = [GroupLayout(page, num_pages)] + ([GroupLayout(page, num_pages, window)] if window else [])
    return CacheManager(groups, max_seqs), np.zeros(4096, dtype=np.int32)


def build(cache, host, entries, vocab=100, max_len=64, budget=64, widths=None):
    return build_step(cache, entries, vocab, max_len, budget, host, widths)


def tables(built, host):
    """The block tables of a built step, one [nseq, width] array per cache group."""
    out, off, n = [], built.layout.off_tables, built.layout.num_seqs
    for w in built.table_widths:
        out.append(host[off:off + n * w].reshape(n, w).tolist())
        off += n * w
    assert off == built.layout.total
    return out


def test_mixed_batch_layout():
    cache, host = make()
    b = build(cache, host, [BatchEntry("a", [5, 6, 7, 8, 9], [4])])
    assert b.first_position == [0] and b.query_lens == [5] and b.seq_start == [0, 5]
    b = build(cache, host, [BatchEntry("a", [10], [0]), BatchEntry("b", [1, 2, 3], [0, 2])])
    L = b.layout
    assert (L.num_tokens, L.num_seqs, L.num_logit_rows, L.max_query_len, L.max_context_len) == (4, 2, 3, 3, 6)
    tok = host[L.off_tokens:L.off_tokens + 4].tolist()
    pos = host[L.off_positions:L.off_positions + 4].tolist()
    seq = host[L.off_seq:L.off_seq + 4].tolist()
    assert (tok, pos, seq) == ([10, 1, 2, 3], [5, 0, 1, 2], [0, 1, 1, 1])
    assert host[L.off_start:L.off_start + 3].tolist() == [0, 1, 4]
    assert host[L.off_context:L.off_context + 2].tolist() == [6, 3]
    assert host[L.off_rows:L.off_rows + 3].tolist() == [0, 1, 3]
    assert host[L.off_slot:L.off_slot + 2].tolist() == [cache.state_slot("a"), cache.state_slot("b")] == b.state_slot
    assert b.table_widths == [2]                               # "a" holds 6 tokens = 2 pages of 4
    table = tables(b, host)[0]
    assert table[0] == cache.block_table("a", 0) and table[1] == cache.block_table("b", 0) + [FREED]
    assert b.first_position == [5, 0]
    cache.check()


def test_fixed_widths_for_graph_replay():
    cache, host = make()
    b = build(cache, host, [BatchEntry("a", [1, 2], [1])], widths=[5])
    assert b.table_widths == [5]
    assert tables(b, host)[0] == [cache.block_table("a", 0) + [FREED] * 4]


def test_windowed_group_gets_its_own_table():
    cache, host = make(window=6)
    build(cache, host, [BatchEntry("a", list(range(10)), [])])
    cache.release_passed("a")
    b = build(cache, host, [BatchEntry("a", [1], [0])])
    (full,), (win,) = tables(b, host)
    assert FREED not in full and win[0] == FREED and win[1:] == cache.block_table("a", 1)[1:]


def test_any_number_of_cache_groups():
    """Twelve groups with pages of different sizes: each gets a table of its own width."""
    pages = [2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 16]
    cache = CacheManager([GroupLayout(p, 64) for p in pages], 3)
    host = np.zeros(8192, dtype=np.int32)
    build(cache, host, [BatchEntry("a", list(range(30)), [])])
    b = build(cache, host, [BatchEntry("b", list(range(7)), [6]), BatchEntry("a", [1], [0])])
    assert b.table_widths == [-(-31 // p) for p in pages]
    for g, table in enumerate(tables(b, host)):
        assert table[1] == cache.block_table("a", g)
        held = cache.block_table("b", g)
        assert table[0] == held + [FREED] * (b.table_widths[g] - len(held))
    cache.check()


@pytest.mark.parametrize("entries, word", [
    ([BatchEntry("a", [1, 100], [])], "out of vocab"),
    ([BatchEntry("a", [-1], [])], "out of vocab"),
    ([BatchEntry("a", [], [])], "no tokens"),
    ([BatchEntry("a", [1, 2], [2])], "wants row"),
    ([BatchEntry("a", [1], []), BatchEntry("a", [2], [])], "twice"),
    ([BatchEntry("a", list(range(65)), [])], "would hold"),
    ([BatchEntry("a", list(range(40)), []), BatchEntry("b", list(range(40)), [])], "max_num_batched_tokens"),
])
def test_refusals_change_nothing(entries, word):
    cache, host = make(num_pages=64)
    with pytest.raises(StepError, match=word):
        build(cache, host, entries)
    assert cache.num_running() == 0 and cache.num_free_pages() == 64 and not cache.has("a")
    cache.check()
    with pytest.raises(StepError, match="at least one"):
        build(cache, host, [])


def test_out_of_pages_and_state_slots():
    cache, host = make(num_pages=4, page=4, max_seqs=2)
    build(cache, host, [BatchEntry("a", list(range(8)), [])])
    with pytest.raises(OutOfPages, match="pools"):
        build(cache, host, [BatchEntry("a", [1], []), BatchEntry("b", list(range(5)), [])])
    assert cache.num_tokens("a") == 8 and not cache.has("b") and cache.num_free_pages() == 2
    build(cache, host, [BatchEntry("b", [1], [])])
    with pytest.raises(OutOfPages, match="state slots"):
        build(cache, host, [BatchEntry("c", [1], [])])
    assert not cache.has("c")
    cache.check()
    cache.free("a"), cache.free("b")
    assert cache.num_free_pages() == 4
