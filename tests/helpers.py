"""Shared pieces of the tests: the two tiny configurations, model folders in a temporary
place, traces for bin/trace_run, and comparison against the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_llama

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 128,
    "tie_word_embeddings": False,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True,
}
# A third one with sizes that are no power of two anywhere and a head size of 48.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 301, "rope_theta": 25000.0,
    "rms_norm_eps": 3e-6, "max_position_embeddings": 512, "tie_word_embeddings": False,
}
CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 5)}

# error of the largest deviation relative to the largest reference logit
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def make_model_folder(path: str, config: dict, seed: int, dtype: str = "float32") -> str:
    from allpaca_b200.weights.random_model import write_random_model
    write_random_model(path, config, seed, dtype, std=0.02, norm_std=0.02)
    return path


def load_weights(path: str) -> Dict[str, torch.Tensor]:
    """Read a model folder with the safetensors package (not the engine's reader)."""
    from safetensors.torch import load_file
    return load_file(os.path.join(path, "model.safetensors"))


def load_config(path: str) -> dict:
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(path: str, tokens: Sequence[int], dtype: str) -> np.ndarray:
    """Logits of the whole sequence from the plain implementation.  For bfloat16 the plain
    implementation computes in float32 and rounds activations where the engine stores them."""
    cfg, w = load_config(path), load_weights(path)
    if dtype == "float32":
        out = plain_llama.llama_forward(cfg, w, tokens, torch.float64)
    else:
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
        out = plain_llama.llama_forward(cfg, w, tokens, torch.float32, round_to=torch.bfloat16)
    return out.to(torch.float64).numpy()


def run_trace(model_dir: str, dtype: str, out_dir: str, steps: List[dict], max_tokens: int,
              extra: Sequence[str] = (), env=None, timeout: int = 900) -> Dict[int, np.ndarray]:
    """Run bin/trace_run as a user would and read back every file it wrote."""
    cfg = load_config(model_dir)
    vocab = cfg["vocab_size"]
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), *extra]
    p = subprocess.run(cmd, input=lines, capture_output=True, text=True, timeout=timeout, env=env)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], p.stdout[-2000:]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        f = os.path.join(out_dir, f"{s['step']}.f32")
        if n == 0:
            assert not os.path.exists(f)
            continue
        arr = np.fromfile(f, dtype="<f4")
        assert arr.size == n * vocab, f"step {s['step']}: {arr.size} floats, expected {n}x{vocab}"
        out[s["step"]] = arr.reshape(n, vocab)
    return out


class TraceBuilder:
    """Collects steps and remembers which (request, position) each output row is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[tuple]] = {}
        self.progress: Dict[str, int] = {}

    def step(self, entries: List[tuple], end: Sequence[str] = ()):
        """entries: (request id, tokens, want) with want relative to this step's tokens."""
        k = len(self.steps)
        rows = []
        es = []
        for rid, toks, want in entries:
            first = self.progress.get(rid, 0)
            for w in want:
                rows.append((rid, first + w))
            self.progress[rid] = first + len(toks)
            es.append({"id": rid, "tokens": list(toks), "want": list(want)})
        for rid in end:
            self.progress.pop(rid, None)
        self.steps.append({"step": k, "entries": es, "end": list(end)})
        self.rows[k] = rows
        return k


def compare(outputs: Dict[int, np.ndarray], builder: TraceBuilder, reference: Dict[str, np.ndarray],
            tol: float, what: str):
    """Every wanted row against the plain logits of (request, position); reports the first
    row that is off, with its place."""
    for k in sorted(builder.rows):
        rows = builder.rows[k]
        if not rows:
            continue
        got = outputs[k]
        for i, (rid, pos) in enumerate(rows):
            ref = reference[rid][pos]
            scale = np.abs(ref).max()
            err = np.abs(got[i].astype(np.float64) - ref).max() / scale
            assert np.isfinite(got[i]).all(), f"{what}: step {k} request {rid} position {pos}: non-finite logits"
            assert err <= tol, (f"{what}: first wrong row at step {k}, request {rid}, position {pos}: "
                                f"error {err:.3e} of the largest logit (tolerance {tol:.1e})")
