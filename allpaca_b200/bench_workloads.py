"""Whole workloads through the Python entry point (scheduler, chunked prompts beside decoding,
sampling, host tokens in and out), with random weights of a named shape:

    python -m allpaca_b200.bench_workloads mixed-1b       # 64 requests, prompts of 16..4096 tokens,
                                                          # 128 new tokens each, portions of 512
    python -m allpaca_b200.bench_workloads batch-13b      # 32 requests, prompts of 1024, 256 new tokens
    python -m allpaca_b200.bench_workloads batch-8b       # 8 requests, prompts of 2048, 256 new tokens

Prints one JSON line: wall time of ``LLM.generate``, generated and prompt tokens a second, the
number of steps the scheduler took and how many requests it preempted.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

WORKLOADS = {
    # name: (preset, requests, (shortest prompt, longest prompt), new tokens, portion, seed)
    "mixed-1b": ("llama-3.2-1b", 64, (16, 4096), 128, 512, 3),
    "batch-13b": ("llama-2-13b", 32, (1024, 1024), 256, 512, 4),
    "batch-8b": ("llama-3.1-8b", 8, (2048, 2048), 256, 2048, 2),
}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m allpaca_b200.bench_workloads")
    p.add_argument("workload", choices=sorted(WORKLOADS))
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    p.add_argument("--requests", type=int, default=0, help="another number of requests (0: the workload's)")
    p.add_argument("--no-graphs", action="store_true")
    p.add_argument("--sampling", choices=["greedy", "default"], default="greedy",
                   help="default: temperature 0.8, top-k 40, top-p 0.95 (the reference's defaults), seeded")
    args = p.parse_args(argv)

    from allpaca_b200.config import EngineConfig
    from allpaca_b200.config.presets import preset_config
    from allpaca_b200.engine.llm import LLM
    from allpaca_b200.engine.runner import ModelRunner
    from allpaca_b200.parts import BuildEnv, Workspace
    from allpaca_b200.sampling.params import SamplingParams
    from allpaca_b200.weights.random_model import random_model_on_device

    preset, nreq, (lo, hi), new_tokens, portion, seed = WORKLOADS[args.workload]
    nreq = args.requests or nreq
    raw = preset_config(preset)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    max_len = hi + new_tokens + 16
    raw["max_position_embeddings"] = max(raw.get("max_position_embeddings", 0), max_len)
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    gen = torch.Generator().manual_seed(seed)
    lengths = [lo if lo == hi else int(torch.randint(lo, hi + 1, (1,), generator=gen)) for _ in range(nreq)]
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    page = 16
    cache_tokens = sum(-(-(n + new_tokens) // page) * page for n in lengths) + 4 * page
    engine = EngineConfig(dtype="bfloat16", page_size=page, max_cache_tokens=cache_tokens, max_num_seqs=nreq,
                          max_num_batched_tokens=max(portion, nreq) + nreq, prefill_chunk=portion,
                          max_model_len=max_len, seed=seed, use_cuda_graphs=not args.no_graphs)
    engine.validate()
    env = BuildEnv(dtype=engine.dtype, device=device, workspace=Workspace(device), page_size=page, max_seqs=nreq)
    cfg, model = random_model_on_device(raw, seed, env)
    runner = ModelRunner(None, engine, model=model, model_config=cfg)
    runner.workspace = env.workspace
    llm = LLM(runner=runner)
    params = SamplingParams.greedy_params(max_tokens=new_tokens) if args.sampling == "greedy" else \
        SamplingParams(max_tokens=new_tokens, seed=seed)

    # a short run first: libraries loaded, graphs of the small batches captured
    llm.generate(prompts[:2], SamplingParams.greedy_params(max_tokens=4))
    torch.cuda.synchronize()
    steps0 = llm.stats["steps"]
    t = time.perf_counter()
    outs = llm.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t
    stats = llm.stats
    generated = sum(len(o.token_ids) for o in outs)
    print(json.dumps({
        "workload": args.workload, "model": preset, "layers": raw["num_hidden_layers"], "layers_in_shape": full_layers,
        "requests": nreq, "prompt_tokens": sum(lengths), "generated_tokens": generated, "seconds": round(wall, 3),
        "generated_tok_s": round(generated / wall, 1), "total_tok_s": round((generated + sum(lengths)) / wall, 1),
        "steps": stats.get("steps", 0) - steps0, "preemptions": stats.get("preemptions", 0),
        "portion": portion, "page_size": page, "sampling": args.sampling, "dtype": "bf16", "data": "synthetic"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
