"""Random workloads through the entry point in 32-bit: requests that arrive while others run,
pools so small that requests are preempted, prompts cut into odd portions, stop tokens,
greedy and seeded sampling.  Every request must end with exactly the tokens it produces when
it runs alone (the 32-bit path does not depend on what else is in a step, and a draw depends
on the request's seed and the token's number only), and the pool must be whole afterwards."""
import random

import pytest

import helpers
from helpers import CONFIGS

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_on_small_pools_match_each_request_alone(tmp_path, seed):
    from allpaca_b200 import LLM, SamplingParams
    rng = random.Random(1000 + seed)
    name = "ABC"[seed % 3]
    config, wseed = CONFIGS[name]
    model = helpers.make_model_folder(str(tmp_path / "m"), config, wseed, "float32")
    vocab, longest_allowed = config["vocab_size"], config["max_position_embeddings"]
    page = rng.choice([4, 8, 16])
    n_req = rng.randint(5, 9)
    requests = []
    for i in range(n_req):
        n_prompt = rng.randint(1, min(70, longest_allowed - 32))
        new = rng.randint(1, 28)
        sampled = rng.random() < 0.5
        params = SamplingParams(
            max_tokens=new, temperature=rng.choice([0.7, 1.1]) if sampled else 0.0,
            top_k=rng.choice([0, 3, 40]) if sampled else 0, top_p=rng.choice([1.0, 0.9]) if sampled else 1.0,
            seed=rng.randint(0, 999), stop_token_ids=[rng.randrange(vocab) for _ in range(rng.choice([0, 0, 6]))])
        requests.append((helpers.random_tokens(n_prompt, vocab, 7000 + 31 * seed + i), params, rng.randint(0, 25)))

    one = LLM(model=model, dtype="float32", page_size=page, max_cache_tokens=256, max_num_seqs=1,
              max_num_batched_tokens=128)
    alone = [one.generate([p], params)[0] for p, params, _ in requests]
    del one

    longest = max(len(p) + params.max_tokens for p, params, _ in requests)
    num_pages = -(-longest // page) + rng.randint(0, 5)
    max_seqs = rng.randint(2, 4)
    llm = LLM(model=model, dtype="float32", page_size=page, num_pages=num_pages, max_num_seqs=max_seqs,
              max_num_batched_tokens=rng.choice([max_seqs + 3, 24, 64]), prefill_chunk=rng.choice([3, 16, 64]))
    done = {}
    step = 0
    waiting = sorted(range(n_req), key=lambda i: requests[i][2])
    while waiting or llm.has_unfinished():
        while waiting and requests[waiting[0]][2] <= step:
            i = waiting.pop(0)
            llm.add_request(requests[i][0], requests[i][1], request_id=i)
        for o in llm.step():
            done[o.request_id] = o
        step += 1
        assert step < 5000, "the workload does not end"
    assert sorted(done) == list(range(n_req))
    for i in range(n_req):
        assert done[i].token_ids == alone[i].token_ids, (i, requests[i][1])
        assert done[i].finish_reason == alone[i].finish_reason
    assert llm.runner.cache.num_running() == 0 and llm.runner.cache.num_free_pages() == num_pages
    llm.runner.cache.check()
