#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of the Llama-3.1-8B shape (preset ``llama-3.1-8b``), random
bfloat16 weights drawn on the device, 8 requests decoding at a context of 4096 tokens.
A step is one decode step of the whole batch.

* ``value``   decoded tokens per second, timed on the device with CUDA events around K steps
              of the step function with next-token choice on the GPU; the chosen tokens reach
              the next step through device memory (``ModelRunner.step(..., device_tokens=)``),
              the step's positions and tables are still built on the host and uploaded;
* ``e2e``     the same through ``LLM.step()`` (scheduler, pinned-memory upload of the step's
              tokens and tables, read-back of the chosen tokens), by the host clock;
* ``prefill`` one prompt of 2048 tokens in one step: tokens/s, ms and the fraction of the
              bf16 peak its FLOPs reach;
* ``roofline`` bytes a decode step must read (every weight once, the cache of the live
              requests) over its time, against the measured HBM copy rate;
* ``points``  decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback
figures measured earlier on the same pool (6650 GB/s, 1590 TFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm() -> int:
    """The reference is a Rust workspace with no Python package; it cannot be installed with
    pip here and neither cargo nor rustc exists to build it."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "spyn/allpaca is a Rust workspace (no setup.py/pyproject): pip install of the "
                      "reference fails offline and no cargo/rustc is present to build it"}))
    return 0


def model_numbers(cfg, layers: int):
    """(linear weight elements used by a step, KV bytes per token, params of the whole model)."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * H + H * cfg.q_size + 3 * I * H
    linear = layers * per_layer + V * H
    kv_per_token = layers * 2 * cfg.kv_size * 2
    return per_layer, linear, kv_per_token


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="llama-3.1-8b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--prefill-only", action="store_true", help="time only the prefill (for profilers)")
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--l2-prefetch-mb", type=int, default=0, help="weight bytes a GEMM may prefetch into L2 early")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (for profilers)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from allpaca_b200 import LLM, SamplingParams, ops
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.config.presets import preset_config
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    from allpaca_b200.engine.scheduler import Request
    from allpaca_b200.ops import library
    from allpaca_b200.parts import BuildEnv, Workspace
    from allpaca_b200.weights.random_model import random_model_on_device

    pk = peaks()
    library.core().ap_gemm_tc_set_l2_prefetch(args.l2_prefetch_mb << 20)
    raw = preset_config(args.preset)
    full_layers = raw["num_hidden_layers"]
    layers = args.layers or full_layers
    raw["num_hidden_layers"] = layers
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    total_steps = args.warmup + args.steps + 8
    max_len = max(args.context, args.prefill_tokens) + 16
    raw["max_position_embeddings"] = max(raw.get("max_position_embeddings", 0), max_len)

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    engine = EngineConfig(dtype="bfloat16", page_size=args.page_size,
                          max_cache_tokens=max_batch * (args.context + args.page_size) + args.prefill_tokens + 64,
                          max_num_seqs=max_batch, max_num_batched_tokens=max(args.prefill_tokens, max_batch),
                          prefill_chunk=args.prefill_tokens, max_model_len=max_len, seed=args.seed,
                          use_cuda_graphs=not args.no_graphs)
    engine.validate()
    env = BuildEnv(dtype=engine.dtype, device=device, workspace=Workspace(device),
                   page_size=engine.page_size, max_seqs=engine.max_num_seqs)
    t0 = time.time()
    cfg, model = random_model_on_device(raw, args.seed, env)
    runner = ModelRunner(None, engine, model=model, model_config=cfg)
    runner.workspace = env.workspace
    torch.cuda.synchronize()
    print(f"[bench] model ready in {time.time() - t0:.1f} s: {layers}/{full_layers} layers, "
          f"cache {runner.memory_report()['cache_bytes'] / 2**30:.1f} GiB", file=sys.stderr, flush=True)
    per_layer, linear_elems, kv_per_token = model_numbers(cfg, layers)
    gen = torch.Generator().manual_seed(args.seed)

    def fast_forward(llm, batch, start_len):
        """Requests that already hold `start_len - 1` tokens of (synthetic, zero) cache: the
        next step runs their last prompt token and decoding goes on from there."""
        ids = []
        for i in range(batch):
            prompt = torch.randint(0, cfg.vocab_size, (start_len,), generator=gen).tolist()
            req = Request(("bench", i), prompt, SamplingParams.greedy_params(max_tokens=10 ** 6))
            llm.scheduler.adopt_running(req, start_len - 1)
            runner.cache.begin(req.request_id)
            runner.cache.append(req.request_id, start_len - 1)
            ids.append(req.request_id)
        return ids

    def drain(llm):
        for req in list(llm.scheduler.running):
            llm.scheduler.abort(req.request_id)
            runner.finish(req.request_id)

    def decode_run(batch, steps, warmup, sample_clocks=False):
        """(device tok/s, ms/step, e2e tok/s, launches, h2d bytes, d2h bytes, clocks)."""
        llm = LLM(runner=runner)
        start_len = args.context - (2 * (warmup + steps) + 2)
        fast_forward(llm, batch, start_len)
        # --- end to end through the entry point, host clock ---
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        t = time.perf_counter()
        for _ in range(steps):
            llm.step()
        llm.flush()                           # the last step's tokens are on the host too
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t
        # --- device-timed steps of the step function with GPU next-token choice ---
        reqs = list(llm.scheduler.running)
        tokens = [r.all_token_ids[-1] for r in reqs]
        for r in reqs:                        # the scheduler no longer drives these requests
            llm.scheduler.abort(r.request_id)
        # the next tokens are chosen on the GPU and handed to the next step on the GPU: no step
        # waits for the host (the end-to-end figure above is the one with host tokens in and out)
        out = torch.tensor(tokens, dtype=torch.int32).to(device)
        entries = [BatchEntry(r.request_id, [0], [0]) for r in reqs]

        def one_step():
            logits = runner.step(entries, device_tokens=out)
            ops.argmax(logits, out)
        for _ in range(warmup):
            one_step()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        calls0 = library.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            one_step()
        stop.record()
        torch.cuda.synchronize()
        tokens = out.tolist()
        ms = start.elapsed_time(stop) / steps
        launches = library.launch_count() - calls0
        clocks = sampler.stop() if sample_clocks else None
        for r in reqs:
            runner.finish(r.request_id)
        h2d = 4 * (3 * batch + (batch + 1) + 3 * batch + batch * -(-args.context // args.page_size))
        return batch / (ms / 1e3), ms, batch * steps / e2e_s, launches, h2d, 4 * batch, clocks

    def prefill_run(tokens_n):
        best = None
        times = []
        for i in range(5):
            prompt = torch.randint(0, cfg.vocab_size, (tokens_n,), generator=gen).tolist()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            runner.step([BatchEntry(("prefill", i), prompt, [tokens_n - 1])])
            stop.record()
            torch.cuda.synchronize()
            runner.finish(("prefill", i))
            ms = start.elapsed_time(stop)
            times.append(round(ms, 3))
            best = ms if best is None or (i > 0 and ms < best) else best
        print(f"[bench] prefill of {tokens_n} tokens, ms per run (the first warms up): {times}", file=sys.stderr, flush=True)
        flops = 2.0 * tokens_n * layers * per_layer + 2.0 * cfg.vocab_size * cfg.hidden_size \
            + layers * 4.0 * cfg.q_size * tokens_n * (tokens_n + 1) / 2
        return best, flops

    if args.prefill_only:
        pms, flops = prefill_run(args.prefill_tokens)
        print(json.dumps({"prefill_ms": round(pms, 3), "tokens": args.prefill_tokens, "layers": layers,
                          "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    value, ms, e2e, launches, h2d, d2h, clocks = decode_run(args.batch, args.steps, args.warmup, True)
    ctx_mid = args.context - (args.steps + 2) // 2
    step_bytes = 2.0 * linear_elems + args.batch * ctx_mid * kv_per_token
    achieved = step_bytes / (ms / 1e3) / 1e9
    result = {
        "metric": f"decode tok/s ({'8B shape' if args.preset == 'llama-3.1-8b' else args.preset}, bf16)", "value": round(value, 2), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": {
            "model": args.preset, "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single-gpu", "layers": layers, "layers_in_shape": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "page_size": args.page_size, "weights": "random N(0,0.02) seed %d" % args.seed,
            "cache_fill": "synthetic (zeros), prefill timed separately",
            "l2": "inputs larger than L2 (weights %.1f GB per step)" % (2.0 * linear_elems / 1e9),
            "peaks": pk["source"],
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }
    if not args.no_points:
        pms, flops = prefill_run(args.prefill_tokens)
        result["prefill"] = {"value": round(args.prefill_tokens / (pms / 1e3), 1), "tokens": args.prefill_tokens,
                             "ms": round(pms, 3),
                             "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                             "of": pk["source"]}
        points = {}
        for b in (1, 64):
            v, _, _, _, _, _, _ = decode_run(b, max(8, args.steps // 4), 3)
            points[f"decode_b{b}"] = round(v, 2)
        result["points"] = points
    ops.check_kernel_status()
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
