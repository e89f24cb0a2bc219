#!/usr/bin/env python3
"""Logits of tiny random Llama models computed with the reference's own CUDA kernels.

The reference's model code is Rust and cannot be compiled where there is no cargo; its CUDA
kernel file can (``baseline/reference_kernels.py``).  This script strings those kernels together
in the order the reference's forward pass does (crates/allpaca-core/src/model.rs:8447-8696 for a
layer, :8759-8791 for the end): embedding row, RMSNorm, the three projections, rotation of Q and
K in the half-split pairing its loader uses for Hugging Face checkpoints (model.rs:7937), causal
grouped-query attention, output projection and residual, RMSNorm, gate and up products, SiLU
times up, down product and residual, final RMSNorm, head.  Every number is produced by the
reference's kernels; only the order of the calls is written here.  The reference has no
llama3 frequency scaling, so the configurations carry none.

Needs a GPU.  Writes ``reference_logits_<name>.npz`` (tokens, float32 logits, the sha256 of the
model.safetensors the weights came from) into ``--out``; the committed copies under
``tests/golden/`` are what ``tests/test_golden.py`` compares the plain implementation with.

    python tests/golden/make_reference_golden.py --out tests/golden
"""
import argparse
import hashlib
import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from golden_configs import GOLDEN, tokens_for  # noqa: E402


def forward(ref, cfg, w, tokens):
    dev = "cuda"
    H, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter, V, eps, theta = cfg["intermediate_size"], cfg["vocab_size"], cfg["rms_norm_eps"], cfg["rope_theta"]
    T = len(tokens)
    w = {k: v.float().to(dev).contiguous() for k, v in w.items()}
    x = torch.empty(T, H, device=dev)
    for t, tok in enumerate(tokens):
        ref.embed_gather(w["model.embed_tokens.weight"], tok, x[t])

    def product(a, name):
        out = torch.empty(a.shape[0], w[name].shape[0], device=dev)
        ref.gemm_nt(a.contiguous(), w[name], out)
        return out

    def norm(a, name):
        out = torch.empty_like(a)
        ref.rmsnorm_rows(a, w[name], out, eps)
        return out
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = norm(x, p + "input_layernorm.weight")
        q = product(h, p + "self_attn.q_proj.weight").view(T, nh, hd)
        k = product(h, p + "self_attn.k_proj.weight").view(T, nkv, hd)
        v = product(h, p + "self_attn.v_proj.weight").view(T, nkv, hd)
        ref.rope_half_split(q, k, 0, theta)
        attn = torch.empty_like(q)
        ref.attention(q, k, v, attn, causal=True)
        o = product(attn.view(T, nh * hd), p + "self_attn.o_proj.weight")
        ref.residual_add(x, o, x)
        h = norm(x, p + "post_attention_layernorm.weight")
        gate, up = product(h, p + "mlp.gate_proj.weight"), product(h, p + "mlp.up_proj.weight")
        act = torch.empty_like(gate)
        ref.silu_mul(gate, up, act)
        d = product(act, p + "mlp.down_proj.weight")
        ref.residual_add(x, d, x)
    h = norm(x, "model.norm.weight")
    head = "lm_head.weight" if "lm_head.weight" in w else "model.embed_tokens.weight"   # tied by absence (model.rs:8006-8009)
    logits = product(h, head)
    torch.cuda.synchronize()
    return logits.cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    from safetensors.torch import load_file
    from allpaca_b200.weights.random_model import write_random_model
    from baseline import reference_kernels
    ref = reference_kernels.load()
    if ref is None:
        sys.exit("the reference's kernels are not built")
    os.makedirs(args.out, exist_ok=True)
    for name, (cfg, seed) in GOLDEN.items():
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, cfg, seed, "float32", std=0.02, norm_std=0.02)
            path = os.path.join(d, "model.safetensors")
            with open(path, "rb") as f:
                sha = hashlib.sha256(f.read()).hexdigest()
            w = load_file(path)
        tokens = tokens_for(name)
        logits = forward(ref, cfg, w, tokens)
        np.savez_compressed(os.path.join(args.out, f"reference_logits_{name}.npz"), tokens=np.asarray(tokens),
                            logits=logits.astype(np.float32), weights_sha256=np.asarray(sha),
                            config=np.asarray(json.dumps(cfg, sort_keys=True)))
        print(name, logits.shape, float(np.abs(logits).max()), sha[:12])


if __name__ == "__main__":
    main()
