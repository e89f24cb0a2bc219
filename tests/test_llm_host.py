"""The entry point's host logic without a GPU: ``LLM`` above a runner that only keeps the
cache manager's books and a sampler whose tokens are a function of (request, position).

What is checked is the interplay the GPU tests reach only by chance: a step kept in flight,
preemption when pages run out, and stop tokens that are seen one step late."""
import random

import pytest

from allpaca_b200.cache import CacheManager, GroupLayout
from allpaca_b200.config import EngineConfig
from allpaca_b200.engine.llm import LLM
from allpaca_b200.sampling import SamplingParams

VOCAB = 1000


def token_at(request_id, position: int) -> int:
    """The token a request's row at ``position`` 'samples' (never below 10, so that small
    numbers are free to serve as stop tokens that a test plants)."""
    return 10 + (hash((str(request_id), position)) % (VOCAB - 10))


class BookkeepingRunner:
    """The step function's effect on the cache manager and nothing else.  Its 'logits' are the
    (request, position) pairs of the wanted rows."""

    def __init__(self, num_pages, page, max_seqs, budget, chunk, max_len):
        self.engine = EngineConfig(dtype="float32", page_size=page, num_pages=num_pages, max_num_seqs=max_seqs,
                                   max_num_batched_tokens=budget, prefill_chunk=chunk, max_model_len=max_len)
        self.engine.validate()
        self.cache = CacheManager([GroupLayout(page, num_pages)], max_seqs)
        self.device = "cpu"
        self.vocab_size = VOCAB
        self.max_model_len = max_len
        self.steps = 0

    def has(self, request) -> bool:
        return self.cache.has(request)

    def finish(self, request) -> None:
        self.cache.free(request)

    def step(self, entries, device_tokens=None):
        rows = []
        for en in entries:
            if not self.cache.has(en.request):
                self.cache.begin(en.request)
            first = self.cache.num_tokens(en.request)
            self.cache.append(en.request, len(en.tokens))
            rows += [(en.request, first + w) for w in en.want]
        self.cache.check()
        self.steps += 1
        return rows


class _Pending:
    def __init__(self, tokens):
        self.tokens = tokens
        self.device = None


class FunctionSampler:
    """Row (request, position) -> ``planted`` token if there is one, else :func:`token_at`."""

    def __init__(self, planted=None):
        self.planted = planted or {}

    def launch(self, logits, params, uniforms):
        return _Pending([self.planted.get(row, token_at(*row)) for row in logits])

    def fetch(self, pending):
        return list(pending.tokens)


def expected(request_id, prompt_len, max_tokens, stops, planted):
    out = []
    for k in range(max_tokens):
        pos = prompt_len + k - 1          # the row that samples the k-th token is the last one held
        t = planted.get((request_id, pos), token_at(request_id, pos))
        out.append(t)
        if t in stops:
            break
    return out


def test_stop_token_of_a_request_preempted_while_its_row_was_in_flight():
    """Six pages of four tokens, two prompts of eight: the young request is preempted when the
    old one needs a page, while the step with the young one's row is in flight; that row's
    token is the young request's stop token.  It must end with what it produced and leave
    the pool whole."""
    runner = BookkeepingRunner(num_pages=6, page=4, max_seqs=4, budget=32, chunk=32, max_len=1000)
    stop = 5
    planted = {("young", 8 + 4 - 1): stop}           # the fifth sampled token
    llm = LLM(runner=runner, sampler=FunctionSampler(planted))
    llm.add_request(list(range(1, 9)), SamplingParams.greedy_params(max_tokens=8), request_id="old")
    llm.add_request(list(range(1, 9)), SamplingParams.greedy_params(max_tokens=8, stop_token_ids=[stop]),
                    request_id="young")
    done = {}
    for _ in range(200):
        for o in llm.step():
            done[o.request_id] = o
        if not llm.has_unfinished():
            break
    assert set(done) == {"old", "young"}
    assert done["young"].token_ids == expected("young", 8, 8, [stop], planted)
    assert done["young"].finish_reason == "stop"
    assert done["old"].token_ids == expected("old", 8, 8, [], planted)
    assert runner.cache.num_free_pages() == 6 and runner.cache.num_running() == 0


@pytest.mark.parametrize("seed", range(40))
def test_random_small_pools_with_stop_tokens(seed):
    """Random workloads on pools so small that requests are preempted, with stop tokens planted
    at random places: every request ends with exactly the tokens its rows produce, and the
    pool is whole afterwards."""
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    n_req = rng.randint(2, 6)
    prompts = [rng.randint(1, 20) for _ in range(n_req)]
    news = [rng.randint(1, 12) for _ in range(n_req)]
    longest = max(p + n for p, n in zip(prompts, news))
    num_pages = -(-longest // page) + rng.randint(0, 3)
    runner = BookkeepingRunner(num_pages=num_pages, page=page, max_seqs=rng.randint(2, 4),
                               budget=rng.choice([8, 16, 32]), chunk=rng.choice([4, 8, 32]), max_len=1000)
    planted, stops = {}, {}
    for i in range(n_req):
        if rng.random() < 0.6:
            stops[i] = [i + 1]                        # below 10: only where planted
            planted[(i, prompts[i] + rng.randint(0, news[i] - 1) - 1)] = i + 1
    llm = LLM(runner=runner, sampler=FunctionSampler(planted))
    for i in range(n_req):
        llm.add_request([1 + (j % 7) for j in range(prompts[i])],
                        SamplingParams.greedy_params(max_tokens=news[i], stop_token_ids=stops.get(i, [])),
                        request_id=i)
    done = {}
    for _ in range(5000):
        for o in llm.step():
            done[o.request_id] = o
        if not llm.has_unfinished():
            break
    assert len(done) == n_req
    for i in range(n_req):
        assert done[i].token_ids == expected(i, prompts[i], news[i], stops.get(i, []), planted), i
    assert runner.cache.num_free_pages() == num_pages and runner.cache.num_running() == 0
