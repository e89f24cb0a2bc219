"""Plain, slow implementation of the dense Llama decoder, used as the oracle.

It rests on the reference's formulas only: the reference's model code is a
Rust workspace and neither cargo nor rustc exists where these tests run, so
it cannot be imported or compiled for a golden comparison.  Every function
cites the reference lines (paths inside the reference project) it restates.

Whole sequences, no cache, one function per part, torch on the CPU.  It
imports nothing from the engine package and takes the raw ``config.json``
dictionary and a ``{tensor name: tensor}`` dictionary in checkpoint names.

``round_to`` emulates a reduced-precision engine: activations are rounded to
that dtype at the places where the engine stores them in it (after a norm,
after a projection that feeds a non-residual consumer, the cached keys and
values, the attention output, the gated activation).  The residual sum,
softmax, norms and rotation angles stay in the compute dtype everywhere.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence

import torch


def _round(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    if round_to is None:
        return x
    return x.to(round_to).to(x.dtype)


# --------------------------------------------------------------------------
# configuration helpers (defaults: crates/allpaca-safetensors/src/sidecar.rs:212-229,
# crates/allpaca-core/src/model.rs:366-372 and :7922)
# --------------------------------------------------------------------------
def sizes(cfg: Mapping) -> dict:
    hidden = cfg.get("hidden_size", 32)
    heads = cfg.get("num_attention_heads", 4)
    kv_heads = cfg.get("num_key_value_heads") or heads
    head_dim = cfg.get("head_dim") or hidden // heads
    return dict(
        hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
        inter=cfg.get("intermediate_size") or 4 * hidden,
        layers=cfg.get("num_hidden_layers", 1), vocab=cfg.get("vocab_size", 32),
        eps=cfg.get("rms_norm_eps", 1e-5), theta=cfg.get("rope_theta", 10000.0),
        tied=bool(cfg.get("tie_word_embeddings") or False),
        scaling=cfg.get("rope_scaling"),
    )


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``ss = sum x^2; inv = 1/sqrt(ss/n + eps); out = x*inv*w``.

    crates/allpaca-cpu/src/kernels.rs:492-507 (eps inside the root, weight
    multiplied last, no ``+1``).
    """
    ss = (x * x).sum(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * inv * weight.to(x.dtype)


def rope_inverse_frequencies(head_dim: int, theta: float,
                             scaling: Optional[Mapping]) -> torch.Tensor:
    """``freq_i = theta^(-i/half)`` for pair ``i`` (crates/allpaca-cpu/src/kernels.rs:517-519),
    then the llama3 rescaling by wavelength.  The reference has no scaling field
    (crates/allpaca-core/src/model.rs:181-274); the rule is the published llama3 one:
    wavelengths shorter than ``n0/high`` are kept, longer than ``n0/low`` are divided
    by ``factor``, and those between are blended linearly in ``n0/wavelength``.
    Computed in float64.
    """
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(float(theta), dtype=torch.float64) ** (-i / half)
    if scaling is None or scaling.get("rope_type", scaling.get("type")) in (None, "default"):
        return freq
    assert scaling.get("rope_type", scaling.get("type")) == "llama3"
    factor = float(scaling["factor"])
    lo = float(scaling.get("low_freq_factor", 1.0))
    hi = float(scaling.get("high_freq_factor", 4.0))
    n0 = float(scaling["original_max_position_embeddings"])
    out = freq.clone()
    for j in range(half):
        wavelen = 2.0 * math.pi / float(freq[j])
        if wavelen < n0 / hi:
            continue
        if wavelen > n0 / lo:
            out[j] = freq[j] / factor
        else:
            s = (n0 / wavelen - lo) / (hi - lo)
            out[j] = (1.0 - s) * freq[j] / factor + s * freq[j]
    return out


def rope_half_split(x: torch.Tensor, positions: torch.Tensor,
                    inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate pairs ``(i, i+half)`` of every head by ``pos * freq_i``.

    Checkpoints in the Hugging Face layout use the half-split pairing
    (crates/allpaca-core/src/model.rs:196-199 and :7937; the rotation itself:
    crates/allpaca-cpu/src/kernels.rs:676-682).  ``x`` is ``[T, heads, head_dim]``.
    """
    half = x.shape[-1] // 2
    angle = positions.to(torch.float64)[:, None] * inv_freq.to(torch.float64)[None, :]
    # the engine forms the angle from a 32-bit frequency table and position
    angle32 = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :])
    if x.dtype == torch.float32:
        angle = angle32.to(torch.float64)
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: Optional[int] = None,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Grouped-query causal attention over one whole sequence.

    ``kv_h = h / (heads/kv_heads)``; score ``= (q.k) * 1/sqrt(head_dim)``; key ``t`` is
    visible to query ``i`` iff ``t <= i`` (and ``i - t < window`` when a window is
    given); softmax by max-subtraction; weighted sum of values.
    crates/allpaca-cpu/src/kernels.rs:318-352 (loop), :327-330 (mask),
    :746-778 (softmax).  ``q``: ``[T, heads, hd]``; ``k, v``: ``[T, kv_heads, hd]``.
    """
    T, heads, hd = q.shape
    kv_heads = k.shape[1]
    reps = heads // kv_heads
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= (idx[:, None] - idx[None, :]) < window
    for h in range(heads):
        kh = k[:, h // reps, :]
        vh = v[:, h // reps, :]
        s = (q[:, h, :] @ kh.T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ vh
    return out


def silu(z: torch.Tensor) -> torch.Tensor:
    """``z / (1 + exp(-z))`` (crates/allpaca-cpu/src/kernels.rs:869-871)."""
    return z / (1.0 + torch.exp(-z))


def swiglu_feed_forward(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                        w_down: torch.Tensor,
                        round_to: Optional[torch.dtype] = None) -> torch.Tensor:
    """``down( silu(gate x) * (up x) )`` (crates/allpaca-core/src/model.rs:5664-5705)."""
    g = _round(x @ w_gate.T, round_to)
    u = _round(x @ w_up.T, round_to)
    a = _round(silu(g) * u, round_to)
    return a @ w_down.T


def attention_mixer(x: torch.Tensor, positions: torch.Tensor, w: Mapping[str, torch.Tensor],
                    prefix: str, s: Mapping, inv_freq: torch.Tensor,
                    round_to: Optional[torch.dtype] = None,
                    window: Optional[int] = None) -> torch.Tensor:
    """Projections, rotation of Q and K (not V), attention, output projection.

    crates/allpaca-core/src/model.rs:8528-8560 (three separate projections, no bias),
    :8573-8604 (rotation at the absolute position), :8639-8667.
    """
    T = x.shape[0]
    q = _round(x @ w[prefix + "q_proj.weight"].T, round_to).view(T, s["heads"], s["head_dim"])
    k = _round(x @ w[prefix + "k_proj.weight"].T, round_to).view(T, s["kv_heads"], s["head_dim"])
    v = _round(x @ w[prefix + "v_proj.weight"].T, round_to).view(T, s["kv_heads"], s["head_dim"])
    q = _round(rope_half_split(q, positions, inv_freq), round_to)
    k = _round(rope_half_split(k, positions, inv_freq), round_to)
    o = _round(causal_attention(q, k, v, window=window), round_to)
    return o.reshape(T, -1) @ w[prefix + "o_proj.weight"].T


def llama_forward(cfg: Mapping, weights: Mapping[str, torch.Tensor],
                  tokens: Sequence[int], dtype: torch.dtype = torch.float32,
                  round_to: Optional[torch.dtype] = None,
                  rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence starting at position 0 (with ``rows``: only of
    those positions, ``[len(rows), vocab]``; everything before the head still runs whole).

    Block order ``x -> norm -> attention -> +x -> norm -> ffn -> +x``
    (crates/allpaca-core/src/model.rs:8447-8696), final norm and head
    (:8759-8791); a missing ``lm_head.weight`` or ``tie_word_embeddings`` uses the
    embedding matrix (:8006-8009).  Tokens must be below the vocabulary size
    (:8215-8219).
    """
    s = sizes(cfg)
    w = {k: t.to(dtype) for k, t in weights.items()}
    toks = torch.as_tensor(list(tokens), dtype=torch.long)
    if toks.numel() and int(toks.max()) >= s["vocab"]:
        raise ValueError(f"token {int(toks.max())} out of vocab {s['vocab']}")
    positions = torch.arange(toks.numel())
    inv_freq = rope_inverse_frequencies(s["head_dim"], s["theta"], s["scaling"])
    if dtype == torch.float32:
        inv_freq = inv_freq.to(torch.float32)
    x = w["model.embed_tokens.weight"][toks]
    for i in range(s["layers"]):
        p = f"model.layers.{i}."
        h = _round(rmsnorm(x, w[p + "input_layernorm.weight"], s["eps"]), round_to)
        x = x + attention_mixer(h, positions, w, p + "self_attn.", s, inv_freq, round_to)
        h = _round(rmsnorm(x, w[p + "post_attention_layernorm.weight"], s["eps"]), round_to)
        x = x + swiglu_feed_forward(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                    w[p + "mlp.down_proj.weight"], round_to)
    h = _round(rmsnorm(x, w["model.norm.weight"], s["eps"]), round_to)
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long)]
    head = w["model.embed_tokens.weight"] if (s["tied"] or "lm_head.weight" not in w) \
        else w["lm_head.weight"]
    return h @ head.T


# --------------------------------------------------------------------------
# sampling (crates/allpaca-core/src/sampling.rs:24-82 and helpers :215-331)
# --------------------------------------------------------------------------
def sample_plain(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                 u: float) -> int:
    """One draw from one row of logits, given the uniform number ``u`` in [0,1).

    ``temperature <= 1e-5`` -> first maximum (sampling.rs:36-38, :215-225); else divide
    by the temperature (:227-234), keep the ``top_k`` largest with ties by token id
    (:238-271; 0 = off), keep the smallest sorted prefix whose probability reaches
    ``top_p`` when ``0 <= top_p < 1`` (:276-309), softmax the survivors (:311-331) and
    walk them subtracting probabilities from ``u`` until it is ``<= 0`` (:55-67).  The
    walk here goes in token-id order, which draws from the same distribution as the
    reference's candidate order.
    """
    l = logits.to(torch.float32).clone()
    if not bool(torch.isfinite(l).any()):
        return 0                              # sampling.rs:37-39
    if temperature <= 1e-5:
        return int(torch.argmax(l))          # torch.argmax returns the first maximum
    l = l / max(temperature, 1e-5)
    ids = [i for i in range(l.numel()) if bool(torch.isfinite(l[i]))]   # sampling.rs:236-244
    V = len(ids)
    order = sorted(ids, key=lambda i: (-float(l[i]), i))
    keep = order
    if top_k and top_k < V:
        keep = order[:top_k]
    if 0.0 <= top_p < 1.0 and len(keep) > 1:
        vals = torch.tensor([float(l[i]) for i in keep], dtype=torch.float32)
        p = torch.exp(vals - vals.max())
        p = p / p.sum()
        acc = 0.0
        cut = len(keep)
        for j in range(len(keep)):
            acc += float(p[j])
            if acc >= top_p:
                cut = j + 1
                break
        keep = keep[:cut]
    keep_sorted = sorted(keep)
    vals = torch.tensor([float(l[i]) for i in keep_sorted], dtype=torch.float32)
    p = torch.exp(vals - vals.max())
    p = p / p.sum()
    r = float(u)
    for j, i in enumerate(keep_sorted):
        r -= float(p[j])
        if r <= 0.0:
            return i
    return keep_sorted[-1]


def greedy_generate(cfg: Mapping, weights: Mapping[str, torch.Tensor], prompt: Sequence[int],
                    max_tokens: int, dtype: torch.dtype = torch.float32,
                    round_to: Optional[torch.dtype] = None) -> list:
    """Greedy continuation by re-running the whole sequence for every new token."""
    toks = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = llama_forward(cfg, weights, toks, dtype, round_to)
        nxt = int(torch.argmax(logits[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
