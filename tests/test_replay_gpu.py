"""bin/trace_run against the plain implementation: the same requests replayed whole, with
the last 32 tokens one by one, in portions of changing size, and mixed with other requests
on a pool so small that pages are used again; in 32-bit and in bfloat16, for three tiny
configurations that differ in every size and option."""
import random

import pytest

import helpers
from helpers import CONFIGS, TOL, TraceBuilder

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [21, 33, 47, 100, 128], "B": [25, 33, 64, 124, 200], "C": [19, 70, 130, 257]}
PORTIONS = [3, 2, 7, 2, 16, 5, 2, 33, 9, 4, 2, 64, 11]


def _round64(n):
    return -(-n // 64) * 64


def build_trace(requests, dense=True):
    """All four modes in one trace; returns (builder, reference ids -> request, max tokens).
    ``dense`` False asks for fewer rows' logits (a large vocabulary makes every row half a
    megabyte): every seventh row and the last of a whole prompt, the ends of a portion."""
    tb = TraceBuilder()
    alias = {}
    peak = 0

    def rows_of(n):
        return list(range(n)) if dense else sorted({0, n - 1} | set(range(0, n, 7)) if n > 16 else {0, n - 1})
    # 1. whole
    for r, toks in requests.items():
        rid = f"w{r}"
        alias[rid] = r
        tb.step([(rid, toks, rows_of(len(toks)))], end=[rid])
        peak = max(peak, _round64(len(toks)))
    # 2. most of it in one step, the last 32 one by one
    for r, toks in requests.items():
        if len(toks) <= 33:
            continue
        rid = f"d{r}"
        alias[rid] = r
        head = len(toks) - 32
        tb.step([(rid, toks[:head], [head - 1])])
        for i in range(head, len(toks)):
            tb.step([(rid, toks[i:i + 1], [0])], end=[rid] if i == len(toks) - 1 else [])
    # 3. portions of changing size, down to two tokens
    for r, toks in requests.items():
        rid = f"p{r}"
        alias[rid] = r
        i = k = 0
        while i < len(toks):
            n = min(PORTIONS[k % len(PORTIONS)], len(toks) - i)
            k += 1
            last = i + n == len(toks)
            tb.step([(rid, toks[i:i + n], rows_of(n))], end=[rid] if last else [])
            i += n
    # 4. mixed: up to four live, portions of some beside decoded tokens of others
    rng = random.Random(1234)
    queue = [f"m{r}" for r in requests] + [f"n{r}" for r in requests]
    for rid in queue:
        alias[rid] = rid[1:]
    live, done_at = [], {}
    while queue or live:
        while queue and len(live) < 4:
            live.append(queue.pop(0))
        peak = max(peak, sum(_round64(len(requests[alias[x]])) for x in live))
        entries, ending = [], []
        for rid in list(live):
            toks = requests[alias[rid]]
            at = tb.progress.get(rid, 0)
            if len(live) > 1 and rng.random() < 0.2 and entries:
                continue                       # left out of this step, goes on later
            if at < int(0.6 * len(toks)):
                n = min(rng.choice([2, 3, 5, 8, 13, 20]), len(toks) - at)
                want = [n - 1] if rng.random() < 0.5 else rows_of(n)
            else:
                n, want = 1, [0]
            entries.append((rid, toks[at:at + n], want))
            if at + n == len(toks):
                ending.append(rid)
                live.remove(rid)
        if entries:
            tb.step(entries, end=ending)
    return tb, alias, peak


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_all_modes(tmp_path, name, dtype):
    config, seed = CONFIGS[name]
    model = helpers.make_model_folder(str(tmp_path / "model"), config, seed, dtype)
    requests = {str(i): helpers.random_tokens(n, config["vocab_size"], 100 + i)
                for i, n in enumerate(LENGTHS[name])}
    tb, alias, peak = build_trace(requests)
    outputs = helpers.run_trace(model, dtype, str(tmp_path / "out"), tb.steps, peak)
    plain = {r: helpers.plain_logits(model, toks, dtype) for r, toks in requests.items()}
    reference = {rid: plain[r] for rid, r in alias.items()}
    helpers.compare(outputs, tb, reference, TOL[dtype], f"config {name} {dtype}")


def test_replay_first_tokens_and_single_token_prompt(tmp_path):
    """The first positions of a sequence, a one-token prompt, and two-token portions."""
    config, seed = CONFIGS["B"]
    model = helpers.make_model_folder(str(tmp_path / "model"), config, seed, "float32")
    toks = helpers.random_tokens(12, config["vocab_size"], 9)
    tb = TraceBuilder()
    tb.step([("one", toks[:1], [0])])
    for k in range(1, 12):
        entries = [("one", toks[k:k + 1], [0])]
        if 2 * (k - 1) < 12:
            entries.append(("two", toks[2 * (k - 1):2 * k], [0, 1]))
        tb.step(entries)
    outputs = helpers.run_trace(model, "float32", str(tmp_path / "out"), tb.steps, 128)
    plain = helpers.plain_logits(model, toks, "float32")
    helpers.compare(outputs, tb, {"one": plain, "two": plain}, TOL["float32"], "first tokens")
