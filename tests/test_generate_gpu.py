"""Generation through the Python entry point and the command line, against the plain
implementation: greedy and seeded temperature sampling, chunked prompts beside decoding,
a pool so small that requests are preempted, long decoding, CUDA graphs on and off."""
import json
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_llama
from helpers import CONFIGS, ROOT

pytestmark = pytest.mark.gpu

# the workloads the benchmark configurations name
WORK = {"A": dict(prompts=[5, 17, 31], new=16, page=16, chunk=512),
        "B": dict(prompts=[1, 9, 40, 100], new=24, page=8, chunk=32)}


def make(tmp_path, name, dtype="float32"):
    config, seed = CONFIGS[name]
    model = helpers.make_model_folder(str(tmp_path / f"model{name}{dtype}"), config, seed, dtype)
    w = WORK.get(name, WORK["A"])
    prompts = [helpers.random_tokens(n, config["vocab_size"], 40 + i) for i, n in enumerate(w["prompts"])]
    return config, model, prompts, w


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_matches_plain_float32(tmp_path, name):
    from allpaca_b200 import LLM, SamplingParams
    config, model, prompts, w = make(tmp_path, name)
    llm = LLM(model=model, dtype="float32", page_size=w["page"], prefill_chunk=w["chunk"],
              max_cache_tokens=1024, max_num_seqs=4, max_num_batched_tokens=128)
    outs = llm.generate(prompts, SamplingParams.greedy_params(max_tokens=w["new"]))
    weights = helpers.load_weights(model)
    for p, o in zip(prompts, outs):
        want = plain_llama.greedy_generate(config, weights, p, w["new"], torch.float32)
        assert o.token_ids == want and o.finish_reason == "length"
        assert o.prompt_tokens == len(p) and o.completion_tokens == w["new"]
    assert llm.runner.cache.num_running() == 0
    assert llm.runner.cache.num_free_pages() == llm.runner.num_pages


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_bfloat16_picks_a_top_token_at_every_step(tmp_path, name):
    from allpaca_b200 import LLM, SamplingParams
    config, model, prompts, w = make(tmp_path, name, "bfloat16")
    llm = LLM(model=model, dtype="bfloat16", page_size=w["page"], prefill_chunk=w["chunk"],
              max_cache_tokens=1024, max_num_seqs=4, max_num_batched_tokens=128)
    outs = llm.generate(prompts, SamplingParams.greedy_params(max_tokens=w["new"]))
    for p, o in zip(prompts, outs):
        full = list(p) + o.token_ids
        logits = helpers.plain_logits(model, full[:-1], "bfloat16")
        for i, tok in enumerate(o.token_ids):
            row = logits[len(p) - 1 + i]
            assert row.max() - row[tok] <= helpers.TOL["bfloat16"] * abs(row).max(), (i, tok, int(row.argmax()))


def test_temperature_sampling_is_seeded_and_follows_the_plain_sampler(tmp_path):
    from allpaca_b200 import LLM, SamplingParams
    from allpaca_b200.sampling import uniform
    config, model, prompts, w = make(tmp_path, "B")
    params = SamplingParams(max_tokens=w["new"], temperature=0.8, top_k=0, top_p=1.0, seed=7)
    runs = []
    for chunk in (32, 7):
        llm = LLM(model=model, dtype="float32", page_size=8, prefill_chunk=chunk, max_cache_tokens=1024,
                  max_num_seqs=4, max_num_batched_tokens=64)
        runs.append([o.token_ids for o in llm.generate(prompts, params)])
    assert runs[0] == runs[1]                    # same seed: same tokens, however prompts were cut
    weights = helpers.load_weights(model)
    off = 0
    for p, toks in zip(prompts, runs[0]):
        full = list(p)
        for n, tok in enumerate(toks):
            logits = plain_llama.llama_forward(config, weights, full, torch.float32)[-1]
            u = uniform(7, n)
            want = plain_llama.sample_plain(logits, 0.8, 0, 1.0, u)
            if tok != want:
                near = {plain_llama.sample_plain(logits, 0.8, 0, 1.0, min(max(u + d, 0.0), 0.999999))
                        for d in (-1e-4, 1e-4)}
                assert tok in near, (n, tok, want)
                off += 1
            full.append(tok)
    assert off <= 2
    other = LLM(model=model, dtype="float32", page_size=8, max_cache_tokens=1024, max_num_seqs=4,
                max_num_batched_tokens=64)
    different = other.generate(prompts, SamplingParams(max_tokens=w["new"], temperature=0.8, top_k=40,
                                                       top_p=0.95, seed=8))
    assert [o.token_ids for o in different] != runs[0]


def test_stop_token_ends_a_reply_and_is_kept(tmp_path):
    from allpaca_b200 import LLM, SamplingParams
    config, model, prompts, w = make(tmp_path, "A")
    llm = LLM(model=model, dtype="float32", max_cache_tokens=512, max_num_seqs=2, max_num_batched_tokens=64)
    free = llm.generate([prompts[1]], SamplingParams.greedy_params(max_tokens=12))[0]
    stop = free.token_ids[5]
    first = free.token_ids.index(stop)
    cut = llm.generate([prompts[1]], SamplingParams.greedy_params(max_tokens=12, stop_token_ids=[stop]))[0]
    assert cut.token_ids == free.token_ids[:first + 1] and cut.finish_reason == "stop"


def test_small_pool_preempts_and_still_matches_each_request_alone(tmp_path):
    from allpaca_b200 import LLM, SamplingParams
    config, model, prompts, w = make(tmp_path, "A")
    prompts = [helpers.random_tokens(n, config["vocab_size"], 70 + i) for i, n in enumerate([30, 28, 33, 25])]
    params = SamplingParams.greedy_params(max_tokens=30)
    alone = []
    for p in prompts:
        llm = LLM(model=model, dtype="float32", page_size=16, max_cache_tokens=128, max_num_seqs=1,
                  max_num_batched_tokens=64)
        alone.append(llm.generate([p], params)[0].token_ids)
    # 4 requests of up to 63 tokens = 4 pages each on a pool of 9 pages: they cannot all fit
    llm = LLM(model=model, dtype="float32", page_size=16, num_pages=9, max_num_seqs=4,
              max_num_batched_tokens=48, prefill_chunk=16)
    outs = llm.generate(prompts, params)
    assert [o.token_ids for o in outs] == alone
    assert llm.stats["preemptions"] > 0 and sum(o.num_preemptions for o in outs) > 0
    assert llm.runner.cache.num_free_pages() == 9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_logits(tmp_path, dtype):
    """400 decode steps from a short prompt (config C takes 512 positions): the logits of
    late positions still match a whole-sequence computation."""
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    config, seed = CONFIGS["C"]
    model = helpers.make_model_folder(str(tmp_path / "m"), config, seed, dtype)
    toks = helpers.random_tokens(420, config["vocab_size"], 11)
    runner = ModelRunner(model, EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=512, max_num_seqs=2,
                                             max_num_batched_tokens=64))
    got = {}
    runner.step([BatchEntry("r", toks[:20], [])])
    for i in range(20, 420):
        logits = runner.step([BatchEntry("r", toks[i:i + 1], [0])])
        if i % 50 == 19 or i >= 410:
            got[i] = logits[0].cpu().double().numpy()
    plain = helpers.plain_logits(model, toks, dtype)
    for i, row in got.items():
        err = abs(row - plain[i]).max() / abs(plain[i]).max()
        assert err <= helpers.TOL[dtype], (i, err)
    # these steps were replayed graphs (all but the first few of each bound on the context), and
    # crossing 256 tokens recorded a second graph for the same batch size (keys: rows, bound on
    # the longest context, bound on the average context)
    recorded = sorted(key for key, g in runner._graphs.items() if g.graph is not None)
    assert recorded == [(1, 256, 256), (1, 512, 512)], recorded
    assert runner.graph_replays >= 390


def test_cuda_graphs_do_not_change_the_tokens(tmp_path):
    from allpaca_b200 import LLM, SamplingParams
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.runner import ModelRunner
    config, model, prompts, w = make(tmp_path, "B", "bfloat16")
    outs = []
    for graphs in (True, False):
        runner = ModelRunner(model, EngineConfig(dtype="bfloat16", page_size=8, max_cache_tokens=1024,
                                                 max_num_seqs=4, max_num_batched_tokens=64, prefill_chunk=32,
                                                 use_cuda_graphs=graphs))
        llm = LLM(runner=runner)
        outs.append([o.token_ids for o in llm.generate(prompts, SamplingParams.greedy_params(max_tokens=24))])
        if graphs:
            # batch sizes that were used three times or more have been recorded
            assert runner._graphs and any(g.graph is not None for g in runner._graphs.values())
    assert outs[0] == outs[1]


def test_command_line_generate(tmp_path):
    config, model, prompts, w = make(tmp_path, "A")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "allpaca"), "generate", "--model", model, "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", " ".join(map(str, prompts[1])),
           "--max-tokens", "6", "--temperature", "0", "--json"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    weights = helpers.load_weights(model)
    assert len(lines) == 2
    for pr, out in zip(prompts[:2], lines):
        assert out["token_ids"] == plain_llama.greedy_generate(config, weights, pr, 6, torch.float32)
        assert out["finish_reason"] == "length" and out["prompt_tokens"] == len(pr)
    syn = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "allpaca"), "generate", "--synthetic", "tiny-b",
                          "--seed", "1", "--prompt-ids", "1 2 3", "--max-tokens", "4"],
                         capture_output=True, text=True, timeout=600)
    assert syn.returncode == 0 and "[length]" in syn.stdout, syn.stderr[-3000:]


def test_checkpoint_with_saved_rotary_buffers_loads(tmp_path):
    """Some exporters save ``rotary_emb.inv_freq`` beside the weights; it is derived from the
    configuration, so it is neither needed nor an error."""
    from safetensors.torch import load_file, save_file
    from allpaca_b200 import LLM, SamplingParams
    config, model, prompts, w = make(tmp_path, "A")
    path = os.path.join(model, "model.safetensors")
    tensors = load_file(path)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    save_file(tensors, path)
    out = LLM(model, dtype="float32").generate(prompts[:1], SamplingParams.greedy_params(max_tokens=3))
    assert len(out[0].token_ids) == 3


@pytest.mark.parametrize("graphs", [True, False])
def test_tokens_handed_over_on_the_device_give_the_same_sequence(tmp_path, graphs):
    """Decoding with the next token chosen on the GPU and read by the next step from device
    memory, without a visit to the host, produces the tokens ``LLM.generate`` produces."""
    from allpaca_b200 import LLM, SamplingParams, ops
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    config, model, prompts, w = make(tmp_path, "B", "bfloat16")
    prompts = prompts[:3]
    new = 20
    engine = EngineConfig(dtype="bfloat16", page_size=8, max_cache_tokens=1024, max_num_seqs=4,
                          max_num_batched_tokens=256, use_cuda_graphs=graphs)
    want = [o.token_ids for o in LLM(runner=ModelRunner(model, engine)).generate(
        prompts, SamplingParams.greedy_params(max_tokens=new))]
    runner = ModelRunner(model, engine)
    out = torch.empty(len(prompts), dtype=torch.int32, device="cuda")
    logits = runner.step([BatchEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)])
    ops.argmax(logits, out)
    got = [out.clone()]
    entries = [BatchEntry(i, [0], [0]) for i in range(len(prompts))]
    for _ in range(new - 1):
        logits = runner.step(entries, device_tokens=out)
        ops.argmax(logits, out)
        got.append(out.clone())
    got = torch.stack(got).T.tolist()
    assert got == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_stop_token_found_one_step_late_changes_no_other_reply(tmp_path, dtype):
    """The step after a stop token is already in flight when the token reaches the host: the
    stopped request's row in it runs for nothing, the other requests go on undisturbed, and a
    request added meanwhile joins them."""
    from allpaca_b200 import LLM, SamplingParams
    config, model, prompts, w = make(tmp_path, "B", dtype)
    kw = dict(model=model, dtype=dtype, page_size=8, max_cache_tokens=1024, max_num_seqs=4,
              max_num_batched_tokens=64, prefill_chunk=32)
    free = LLM(**kw).generate(prompts[:3], SamplingParams.greedy_params(max_tokens=20))
    stops = [free[0].token_ids[4], free[2].token_ids[11]]
    params = [SamplingParams.greedy_params(max_tokens=20, stop_token_ids=[stops[0]]),
              SamplingParams.greedy_params(max_tokens=20),
              SamplingParams.greedy_params(max_tokens=20, stop_token_ids=[stops[1]])]
    llm = LLM(**kw)
    ids = [llm.add_request(p, sp) for p, sp in zip(prompts[:3], params)]
    done = {}
    steps = 0
    late = None
    while llm.has_unfinished():
        for o in llm.step():
            done[o.request_id] = o
        steps += 1
        if steps == 8:
            late = llm.add_request(prompts[3], SamplingParams.greedy_params(max_tokens=6))
    for o in llm.flush():
        done[o.request_id] = o
    cut0 = free[0].token_ids[:free[0].token_ids.index(stops[0]) + 1]
    cut2 = free[2].token_ids[:free[2].token_ids.index(stops[1]) + 1]
    assert done[ids[0]].token_ids == cut0 and done[ids[0]].finish_reason == "stop"
    assert done[ids[1]].token_ids == free[1].token_ids and done[ids[1]].finish_reason == "length"
    assert done[ids[2]].token_ids == cut2 and done[ids[2]].finish_reason == "stop"
    alone = LLM(**kw).generate([prompts[3]], SamplingParams.greedy_params(max_tokens=6))[0]
    assert done[late].token_ids == alone.token_ids
    assert llm.runner.cache.num_running() == 0
    llm.runner.cache.check()
