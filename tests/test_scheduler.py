"""The scheduler's decisions: admission, token budget, portions, finishing, and what happens
when pages run out.  The step function is replaced by bookkeeping on the cache manager."""
import pytest

from allpaca_b200.cache import CacheManager, GroupLayout
from allpaca_b200.engine import AdmissionError, FinishReason, Request, Scheduler
from allpaca_b200.sampling import SamplingParams


def make(num_pages=64, page=4, max_seqs=4, budget=16, chunk=8, max_len=1000):
    cache = CacheManager([GroupLayout(page, num_pages)], max_seqs)
    return cache, Scheduler(cache, max_seqs, budget, chunk, max_len)


def run_step(cache, sched, next_token=lambda req: 7):
    out = sched.schedule()
    for r in out.rows:
        if not cache.has(r.request.request_id):
            cache.begin(r.request.request_id)
        assert cache.num_tokens(r.request.request_id) == r.start
        cache.append(r.request.request_id, r.count)
    cache.check()
    sampled = {r.request.request_id: next_token(r.request) for r in out.rows if r.samples}
    finished = sched.advance(out, sampled)
    for f in finished:
        cache.free(f.request_id)
    return out, finished


def req(i, n, max_tokens=4, stop=()):
    return Request(i, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, temperature=0,
                                                            stop_token_ids=list(stop)))


def test_prompt_is_cut_into_portions_under_budget_and_chunk():
    cache, s = make(budget=16, chunk=8)
    s.add(req("a", 21))
    counts = []
    for _ in range(3):
        out, _ = run_step(cache, s)
        counts.append([(r.start, r.count, r.samples) for r in out.rows])
    assert counts == [[(0, 8, False)], [(8, 8, False)], [(16, 5, True)]]
    out, _ = run_step(cache, s)
    assert [(r.start, r.count, r.samples) for r in out.rows] == [(21, 1, True)]


def test_decodes_come_first_and_share_the_step_with_a_prompt_portion():
    cache, s = make(budget=10, chunk=8)
    s.add(req("a", 3))
    run_step(cache, s)                       # a: prompt done, one token sampled
    s.add(req("b", 20))
    out, _ = run_step(cache, s)
    assert [(r.request.request_id, r.count) for r in out.rows] == [("a", 1), ("b", 8)]
    out, _ = run_step(cache, s)
    assert [(r.request.request_id, r.count) for r in out.rows] == [("a", 1), ("b", 8)]
    assert out.num_tokens <= 10


def test_budget_is_shared_between_prompts_in_arrival_order():
    cache, s = make(budget=12, chunk=8)
    s.add(req("a", 30)), s.add(req("b", 30))
    out, _ = run_step(cache, s)
    assert [(r.request.request_id, r.count) for r in out.rows] == [("a", 8), ("b", 4)]


def test_max_num_seqs_limits_admission():
    cache, s = make(max_seqs=2, budget=64, chunk=64)
    for i in range(3):
        s.add(req(i, 4, max_tokens=2))
    out, _ = run_step(cache, s)
    assert [r.request.request_id for r in out.rows] == [0, 1]
    out, fin = run_step(cache, s)            # both produce their second token and finish
    assert sorted(f.request_id for f in fin) == [0, 1]
    out, _ = run_step(cache, s)
    assert [r.request.request_id for r in out.rows] == [2]


def test_finish_reasons_and_stop_token_is_kept():
    cache, s = make()
    s.add(req("len", 2, max_tokens=3))
    s.add(req("stop", 2, max_tokens=10, stop=[99]))
    toks = {"len": iter([5, 6, 7, 8]), "stop": iter([5, 99, 1])}
    done = {}
    while s.has_unfinished():
        _, fin = run_step(cache, s, lambda r: next(toks[r.request_id]))
        done.update({f.request_id: f for f in fin})
    assert done["len"].output_token_ids == [5, 6, 7] and done["len"].finish_reason == FinishReason.LENGTH
    assert done["stop"].output_token_ids == [5, 99] and done["stop"].finish_reason == FinishReason.STOP
    assert cache.num_free_pages() == 64 and cache.num_running() == 0


def test_stop_wins_over_length_and_model_length_ends_a_request():
    cache, s = make(max_len=6)
    s.add(req("a", 2, max_tokens=1, stop=[7]))
    s.add(req("b", 4, max_tokens=50))
    done = {}
    while s.has_unfinished():
        _, fin = run_step(cache, s)
        done.update({f.request_id: f for f in fin})
    assert done["a"].finish_reason == FinishReason.STOP
    assert done["b"].finish_reason == FinishReason.LENGTH and len(done["b"].output_token_ids) == 2


def test_requests_that_can_never_fit_are_refused():
    cache, s = make(num_pages=4, page=4, max_len=100)
    with pytest.raises(AdmissionError, match="pages"):
        s.add(req("big", 10, max_tokens=10))
    with pytest.raises(AdmissionError, match="at least one"):
        s.add(Request("e", [], SamplingParams()))
    _, s2 = make(max_len=8)
    with pytest.raises(AdmissionError, match="length limit"):
        s2.add(req("long", 8))


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 4 tokens; two requests that each grow to 16 tokens = 4 pages
    cache, s = make(num_pages=6, page=4, budget=32, chunk=32)
    s.add(req("old", 8, max_tokens=8))
    s.add(req("young", 8, max_tokens=8))
    preempted_seen = False
    done = {}
    steps = 0
    while s.has_unfinished():
        out, fin = run_step(cache, s)
        steps += 1
        assert steps < 200
        if out.preempted:
            preempted_seen = True
            assert [p.request_id for p in out.preempted] == ["young"]
            assert not cache.has("young")
            young = out.preempted[0]
            assert young.num_computed == 0 and s.waiting[0] is young
        done.update({f.request_id: f for f in fin})
    assert preempted_seen
    assert len(done["old"].output_token_ids) == 8 and len(done["young"].output_token_ids) == 8
    assert done["young"].num_preemptions >= 1 and done["old"].num_preemptions == 0
    assert cache.num_free_pages() == 6


def test_recompute_keeps_the_tokens_already_produced():
    cache, s = make(num_pages=6, page=4, budget=32, chunk=32)
    s.add(req("old", 8, max_tokens=8)), s.add(req("young", 8, max_tokens=8))
    counter = {"old": 100, "young": 200}

    def tok(r):
        counter[r.request_id] += 1
        return counter[r.request_id]
    done = {}
    while s.has_unfinished():
        out, fin = run_step(cache, s, tok)
        for r in out.rows:
            if r.request.num_preemptions and r.start == 0:
                # the recomputation runs prompt and produced tokens together as one prompt
                assert r.request.num_tokens == 8 + len(r.request.output_token_ids)
        done.update({f.request_id: f for f in fin})
    assert done["young"].output_token_ids == list(range(201, 209))
    assert done["old"].output_token_ids == list(range(101, 109))


def test_many_requests_on_a_small_pool_all_finish():
    cache, s = make(num_pages=10, page=4, max_seqs=4, budget=24, chunk=8)
    for i in range(12):
        s.add(req(i, 3 + (i * 5) % 17, max_tokens=2 + i % 7))
    done = {}
    steps = 0
    while s.has_unfinished():
        out, fin = run_step(cache, s)
        assert out.num_tokens <= 24
        steps += 1
        assert steps < 2000
        done.update({f.request_id: f for f in fin})
    assert len(done) == 12
    for i in range(12):
        assert len(done[i].output_token_ids) == 2 + i % 7
    assert cache.num_free_pages() == 10 and cache.num_running() == 0


def test_abort_removes_a_request():
    cache, s = make()
    s.add(req("a", 5)), s.add(req("b", 5))
    run_step(cache, s)
    r = s.abort("a")
    cache.free("a")
    assert r.request_id == "a" and [x.request_id for x in s.running] == ["b"]
    assert s.abort("zzz") is None


def test_token_slice_equals_slicing_the_joined_list():
    from allpaca_b200.engine.scheduler import Request
    from allpaca_b200.sampling.params import SamplingParams
    req = Request("r", [1, 2, 3, 4, 5], SamplingParams())
    req.output_token_ids = [6, 7, 8]
    for start in range(0, 9):
        for count in range(0, 9 - start):
            assert req.token_slice(start, count) == req.all_token_ids[start:start + count]


def test_two_halves_of_advance_with_a_step_in_flight():
    """The next step is planned before the tokens of the step before are known: a request at its
    length limit is planned no more, a stop token is found one step late, the row planned in
    between runs for nothing and its token is dropped."""
    cache, s = make(budget=16, chunk=8)
    a, b = req("a", 3, max_tokens=5, stop=[99]), req("b", 3, max_tokens=2)
    s.add(a), s.add(b)

    def run(out):
        for r in out.rows:
            if r.request.status.value == "finished":
                continue                                  # its cache is gone: the caller drops the row
            if not cache.has(r.request.request_id):
                cache.begin(r.request.request_id)
            cache.append(r.request.request_id, r.count)

    out0 = s.schedule()
    run(out0)
    s.advance_counts(out0)
    out1 = s.schedule()                                   # planned without the tokens of step 0
    assert [(r.request.request_id, r.start, r.count) for r in out1.rows] == [("a", 3, 1), ("b", 3, 1)]
    assert s.resolve(out0, [7, 7]) == []
    run(out1)
    s.advance_counts(out1)                                # b now holds max_tokens tokens
    out2 = s.schedule()
    assert [r.request.request_id for r in out2.rows] == ["a"]
    done = s.resolve(out1, [99, 8])
    assert {d.request_id: d.finish_reason for d in done} == {"a": FinishReason.STOP, "b": FinishReason.LENGTH}
    for d in done:
        cache.free(d.request_id)
    run(out2)
    s.advance_counts(out2)
    assert s.has_unfinished()                             # step 2 is still to be resolved
    assert s.resolve(out2, [5]) == [] and not s.has_unfinished()
    assert a.output_token_ids == [7, 99] and b.output_token_ids == [7, 8]
    assert cache.num_running() == 0 and cache.num_free_pages() == 64
    assert s.schedule().rows == []


def test_windowed_group_admits_a_prompt_longer_than_its_pool():
    """A group with a window gives back the pages the window has passed, so a prompt longer than
    the whole pool is accepted by add() and must then be admitted and run to its end: admission
    asks for what the request holds at once, not for every token it will ever see."""
    page, num_pages, window = 4, 12, 8
    cache = CacheManager([GroupLayout(page, num_pages, window)], 4)
    s = Scheduler(cache, 4, 16, 8, 1000)
    s.add(req("long", 100, max_tokens=6))
    s.add(req("second", 30, max_tokens=3))
    done = {}
    steps = 0
    while s.has_unfinished():
        out = s.schedule()
        assert out.rows, "nothing was planned although requests are pending"
        for r in out.rows:
            if not cache.has(r.request.request_id):
                cache.begin(r.request.request_id)
            cache.append(r.request.request_id, r.count)
            cache.release_passed(r.request.request_id)
        cache.check()
        fin = s.advance(out, {r.request.request_id: 7 for r in out.rows if r.samples})
        for f in fin:
            cache.free(f.request_id)
            done[f.request_id] = f
        steps += 1
        assert steps < 500
    assert len(done["long"].output_token_ids) == 6 and len(done["second"].output_token_ids) == 3
    assert cache.num_free_pages() == num_pages and cache.num_running() == 0
