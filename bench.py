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
* ``prefill`` one prompt of 2048 tokens in one step: tokens/s, the best time of five runs (``ms``)
              and their median (``median_ms``: repeated back to back the runs slow down as the
              power cap pulls the clock down), and the fractions of the bf16 peak their FLOPs reach;
* ``roofline`` bytes a decode step must read (every weight once, the cache of the live
              requests) over its time, against the measured HBM copy rate;
* ``points``  decode at batch 1, 64 and 128, and at batch 8 of the other benchmark shapes
              (``--no-presets`` leaves those out), each with its fraction of the copy rate;
* ``clocks``  SM clocks and throttle reasons sampled by nvidia-smi across the timed regions.
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
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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


class Workbench:
    """One model shape with random weights on the device, its runner, and the timed runs."""

    def __init__(self, preset: str, layers, args, max_batch: int):
        import torch
        from allpaca_b200.config import EngineConfig
        from allpaca_b200.config.presets import preset_config
        from allpaca_b200.engine.runner import ModelRunner
        from allpaca_b200.parts import BuildEnv, Workspace
        from allpaca_b200.weights.random_model import random_model_on_device
        self.torch, self.args, self.preset = torch, args, preset
        raw = preset_config(preset)
        self.full_layers = raw["num_hidden_layers"]
        self.layers = layers or self.full_layers
        raw["num_hidden_layers"] = self.layers
        max_len = max(args.context, args.prefill_tokens) + 16
        raw["max_position_embeddings"] = max(raw.get("max_position_embeddings", 0), max_len)
        self.device = torch.device("cuda:0")
        torch.cuda.set_device(self.device)
        engine = EngineConfig(dtype="bfloat16", page_size=args.page_size,
                              max_cache_tokens=max_batch * (args.context + args.page_size) + args.prefill_tokens + 64,
                              max_num_seqs=max_batch, max_num_batched_tokens=max(args.prefill_tokens, max_batch),
                              prefill_chunk=args.prefill_tokens, max_model_len=max_len, seed=args.seed,
                              use_cuda_graphs=not args.no_graphs)
        engine.validate()
        env = BuildEnv(dtype=engine.dtype, device=self.device, workspace=Workspace(self.device),
                       page_size=engine.page_size, max_seqs=engine.max_num_seqs)
        t0 = time.time()
        self.cfg, model = random_model_on_device(raw, args.seed, env)
        self.runner = ModelRunner(None, engine, model=model, model_config=self.cfg)
        self.runner.workspace = env.workspace
        torch.cuda.synchronize()
        print(f"[bench] {preset} ready in {time.time() - t0:.1f} s: {self.layers}/{self.full_layers} layers, "
              f"cache {self.runner.memory_report()['cache_bytes'] / 2**30:.1f} GiB", file=sys.stderr, flush=True)
        self.per_layer, self.linear_elems, self.kv_per_token = model_numbers(self.cfg, self.layers)
        self.gen = torch.Generator().manual_seed(args.seed)

    def close(self):
        self.runner = None
        import gc
        gc.collect()
        self.torch.cuda.empty_cache()

    def _fast_forward(self, llm, batch, start_len):
        """Requests that already hold `start_len - 1` tokens of (synthetic, zero) cache: the
        next step runs their last prompt token and decoding goes on from there."""
        from allpaca_b200 import SamplingParams
        from allpaca_b200.engine.scheduler import Request
        for i in range(batch):
            prompt = self.torch.randint(0, self.cfg.vocab_size, (start_len,), generator=self.gen).tolist()
            req = Request(("bench", i), prompt, SamplingParams.greedy_params(max_tokens=10 ** 6))
            llm.scheduler.adopt_running(req, start_len - 1)
            self.runner.cache.begin(req.request_id)
            self.runner.cache.append(req.request_id, start_len - 1)

    def decode_run(self, batch, steps, warmup, sample_clocks=False):
        """(device tok/s, ms/step, e2e tok/s, launches, h2d bytes, d2h bytes, clocks)."""
        torch, runner, args = self.torch, self.runner, self.args
        from allpaca_b200 import LLM, ops
        from allpaca_b200.engine.batch import BatchEntry
        from allpaca_b200.ops import library
        llm = LLM(runner=runner)
        start_len = args.context - (2 * (warmup + steps) + 2)
        self._fast_forward(llm, batch, start_len)
        # the clocks are sampled over both timed regions (the same K steps twice: through the
        # entry point, then device-timed)
        sampler = ClockSampler()
        # --- end to end through the entry point, host clock ---
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        if sample_clocks:
            sampler.start()
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
        out = torch.tensor(tokens, dtype=torch.int32).to(self.device)
        entries = [BatchEntry(r.request_id, [0], [0]) for r in reqs]

        def one_step():
            logits = runner.step(entries, device_tokens=out)
            ops.argmax(logits, out)
        for _ in range(warmup):
            one_step()
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

    def step_bytes(self, batch, steps):
        """What a decode step has to read: every weight once, and the cache of the live requests
        at the middle of the timed region."""
        ctx_mid = self.args.context - (steps + 2) // 2
        return 2.0 * self.linear_elems + batch * ctx_mid * self.kv_per_token

    def prefill_run(self, tokens_n):
        """(best ms, median ms, flops) of five prompts of ``tokens_n`` tokens, after one that warms up and a
        second of rest."""
        torch, runner, cfg = self.torch, self.runner, self.cfg
        from allpaca_b200.engine.batch import BatchEntry
        times = []
        for i in range(6):
            prompt = torch.randint(0, cfg.vocab_size, (tokens_n,), generator=self.gen).tolist()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            runner.step([BatchEntry(("prefill", i), prompt, [tokens_n - 1])])
            stop.record()
            torch.cuda.synchronize()
            runner.finish(("prefill", i))
            times.append(round(start.elapsed_time(stop), 3))
            if i == 0:
                # the GPU comes here from the decode runs at the clock the power cap left it: a second of
                # rest, so that the first timed run shows the burst clock (the peak it is set against is a
                # burst figure too); the five runs follow one another at once, and their median shows
                # what the power cap allows in the long run
                time.sleep(1.0)
        print(f"[bench] prefill of {tokens_n} tokens, ms per run (the first warms up): {times}", file=sys.stderr, flush=True)
        flops = 2.0 * tokens_n * self.layers * self.per_layer + 2.0 * cfg.vocab_size * cfg.hidden_size \
            + self.layers * 4.0 * cfg.q_size * tokens_n * (tokens_n + 1) / 2
        return min(times[1:]), statistics.median(times[1:]), flops


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="llama-3.1-8b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--no-presets", action="store_true",
                    help="skip the decode points of the other benchmark shapes (Llama-3.2-1B, Llama-2-13B)")
    ap.add_argument("--prefill-only", action="store_true", help="time only the prefill (for profilers)")
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (for profilers)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if 2 * (args.warmup + args.steps) + 66 > args.context:
        print(f"bench.py: --steps {args.steps} does not fit a context of {args.context} tokens twice over "
              f"(the steps run once through the entry point and once device-timed)", file=sys.stderr)
        return 2

    from allpaca_b200 import ops
    pk = peaks()
    max_batch = args.batch if args.no_points else max(args.batch, 128)
    bench = Workbench(args.preset, args.layers, args, max_batch)
    cfg, layers = bench.cfg, bench.layers
    if args.prefill_only:
        pms, pmed, flops = bench.prefill_run(args.prefill_tokens)
        print(json.dumps({"prefill_ms": round(pms, 3), "median_ms": round(pmed, 3), "tokens": args.prefill_tokens,
                          "layers": layers, "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    value, ms, e2e, launches, h2d, d2h, clocks = bench.decode_run(args.batch, args.steps, args.warmup, True)
    achieved = bench.step_bytes(args.batch, args.steps) / (ms / 1e3) / 1e9
    result = {
        "metric": f"decode tok/s ({'8B shape' if args.preset == 'llama-3.1-8b' else args.preset}, bf16)", "value": round(value, 2), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": {
            "model": args.preset, "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single-gpu", "layers": layers, "layers_in_shape": bench.full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "page_size": args.page_size, "weights": "random N(0,0.02) seed %d" % args.seed,
            "cache_fill": "synthetic (zeros), prefill timed separately",
            "l2": "inputs larger than L2 (weights %.1f GB per step)" % (2.0 * bench.linear_elems / 1e9),
            "peaks": pk["source"],
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }
    if not args.no_points:
        pms, pmed, flops = bench.prefill_run(args.prefill_tokens)
        result["prefill"] = {"value": round(args.prefill_tokens / (pms / 1e3), 1), "tokens": args.prefill_tokens,
                             "ms": round(pms, 3), "median_ms": round(pmed, 3),
                             "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                             "frac_median": round(flops / (pmed / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                             "of": pk["source"]}
        points = {}
        side_steps = max(8, min(args.steps // 4, 64))
        for b in (1, 64, 128):
            v, bms, _, _, _, _, _ = bench.decode_run(b, side_steps, 3)
            points[f"decode_b{b}"] = round(v, 2)
            points[f"decode_b{b}_hbm_frac"] = round(bench.step_bytes(b, side_steps) / (bms / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        if not args.no_presets and args.preset == "llama-3.1-8b" and args.layers is None:
            # the other benchmark shapes, full size, the same batch and context
            ops.check_kernel_status()
            bench.close()
            for other in ("llama-3.2-1b", "llama-2-13b"):
                wb = Workbench(other, None, args, args.batch)
                v, bms, _, _, _, _, _ = wb.decode_run(args.batch, side_steps, 3)
                points[f"decode_b{args.batch}_{other}"] = round(v, 2)
                points[f"decode_b{args.batch}_{other}_hbm_frac"] = round(
                    wb.step_bytes(args.batch, side_steps) / (bms / 1e3) / 1e9 / pk["hbm_gbs"], 4)
                wb.close()
        result["points"] = points
    ops.check_kernel_status()
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
