"""The plain implementation itself, the sampling options and the uniform numbers (no GPU)."""
import math

import pytest
import torch

import helpers
import plain_llama as pl
from allpaca_b200.parts.rope import inverse_frequencies
from allpaca_b200.sampling import SamplingParams, uniform


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = pl.rmsnorm(x, w, 1e-5)
    inv = 1 / math.sqrt((9 + 16) / 2 + 1e-5)
    assert torch.allclose(out, torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=torch.float64))


def test_rope_is_a_rotation_of_half_split_pairs():
    inv = pl.rope_inverse_frequencies(8, 10000.0, None)
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    pos = torch.arange(5)
    y = pl.rope_half_split(x, pos, inv)
    assert torch.allclose(y[0], x[0])                                    # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    a = 3 * float(inv[1])
    assert torch.allclose(y[3, 0, 1], x[3, 0, 1] * math.cos(a) - x[3, 0, 5] * math.sin(a))
    assert torch.allclose(y[3, 0, 5], x[3, 0, 1] * math.sin(a) + x[3, 0, 5] * math.cos(a))
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s = lambda m, n: float((pl.rope_half_split(q, torch.tensor([m]), inv) *      # noqa: E731
                            pl.rope_half_split(k, torch.tensor([n]), inv)).sum())
    assert abs(s(7, 3) - s(14, 10)) < 1e-9


def test_llama3_scaling_regimes_and_engine_table_agree():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = pl.rope_inverse_frequencies(32, 500000.0, None)
    scaled = pl.rope_inverse_frequencies(32, 500000.0, sc)
    wavelen = 2 * math.pi / base
    short, long_ = wavelen < 64 / 4, wavelen > 64 / 1
    assert short.any() and long_.any() and (~short & ~long_).any()     # all three regimes occur
    assert torch.equal(scaled[short], base[short])
    assert torch.allclose(scaled[long_], base[long_] / 8)
    mid = ~short & ~long_
    assert ((scaled[mid] < base[mid]) & (scaled[mid] > base[mid] / 8)).all()
    engine = inverse_frequencies(32, 500000.0, {k: v for k, v in sc.items() if k != "rope_type"})
    assert torch.allclose(engine, scaled, rtol=1e-14)


def test_causal_attention_mask_groups_and_window():
    T, heads, kvh, hd = 6, 4, 2, 4
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, heads, hd, generator=g, dtype=torch.float64)
    k = torch.randn(T, kvh, hd, generator=g, dtype=torch.float64)
    v = torch.randn(T, kvh, hd, generator=g, dtype=torch.float64)
    o = pl.causal_attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])   # head h reads kv head h//2
    s = (q[2, 1] @ k[:3, 0].T) / math.sqrt(hd)
    assert torch.allclose(o[2, 1], torch.softmax(s, 0) @ v[:3, 0])
    assert torch.allclose(pl.causal_attention(q, k, v, window=1)[4, 2], v[4, 1])   # sees itself only
    w2 = pl.causal_attention(q, k, v, window=2)
    s = (q[5, 0] @ k[4:6, 0].T) / math.sqrt(hd)
    assert torch.allclose(w2[5, 0], torch.softmax(s, 0) @ v[4:6, 0])


def test_forward_is_causal_and_tying_follows_flag_or_absence(tmp_path):
    cfg, seed = helpers.CONFIGS["A"]
    model = helpers.make_model_folder(str(tmp_path / "a"), cfg, seed)
    w = helpers.load_weights(model)
    toks = helpers.random_tokens(12, cfg["vocab_size"], 1)
    full = pl.llama_forward(cfg, w, toks, torch.float64)
    part = pl.llama_forward(cfg, w, toks[:7], torch.float64)
    assert torch.allclose(full[:7], part, atol=1e-12)                    # later tokens change nothing earlier
    f32 = pl.llama_forward(cfg, w, toks, torch.float32)
    assert float((f32.double() - full).abs().max() / full.abs().max()) < 1e-5
    untied = dict(w)
    tied = {k: v for k, v in w.items() if k != "lm_head.weight"}
    assert not torch.allclose(pl.llama_forward(cfg, tied, toks, torch.float64), full)
    emb_head = dict(w, **{"lm_head.weight": w["model.embed_tokens.weight"]})
    assert torch.allclose(pl.llama_forward(cfg, tied, toks, torch.float64),
                          pl.llama_forward(cfg, emb_head, toks, torch.float64))
    assert torch.allclose(pl.llama_forward(dict(cfg, tie_word_embeddings=True), untied, toks, torch.float64),
                          pl.llama_forward(cfg, tied, toks, torch.float64))
    with pytest.raises(ValueError, match="out of vocab"):
        pl.llama_forward(cfg, w, [cfg["vocab_size"]])


def test_bfloat16_emulation_differs_but_stays_close(tmp_path):
    cfg, seed = helpers.CONFIGS["B"]
    model = helpers.make_model_folder(str(tmp_path / "b"), cfg, seed, "bfloat16")
    toks = helpers.random_tokens(30, cfg["vocab_size"], 2)
    exact, rounded = helpers.plain_logits(model, toks, "float32"), helpers.plain_logits(model, toks, "bfloat16")
    err = abs(exact - rounded).max() / abs(exact).max()
    assert 1e-4 < err < helpers.TOL["bfloat16"]


def test_sample_plain_options():
    logits = torch.tensor([1.0, 3.0, 3.0, -1.0, float("-inf"), 2.0])
    assert pl.sample_plain(logits, 0.0, 0, 1.0, 0.9) == 1                 # greedy: first maximum
    assert pl.sample_plain(logits, 1.0, 1, 1.0, 0.99) == 1                # top_k 1, tie to the lower id
    assert pl.sample_plain(logits, 1.0, 2, 1.0, 0.99) == 2                # the two 3.0s survive
    assert pl.sample_plain(logits, 1.0, 0, 0.0, 0.99) == 1                # top_p 0 keeps the first only
    p = torch.softmax(logits[[0, 1, 2, 3, 5]], 0)
    assert pl.sample_plain(logits, 1.0, 0, 1.0, float(p[0]) - 1e-6) == 0
    assert pl.sample_plain(logits, 1.0, 0, 1.0, float(p[0]) + 1e-6) == 1
    assert pl.sample_plain(logits, 1.0, 0, 1.0, 0.999999) == 5            # never the -inf entry
    assert pl.sample_plain(torch.full((4,), float("-inf")), 1.0, 0, 1.0, 0.5) == 0
    # top_p keeps the smallest prefix that reaches p: 3.0, 3.0 carry 0.39 each
    assert {pl.sample_plain(logits, 1.0, 0, 0.5, u) for u in (0.0, 0.3, 0.6, 0.99)} == {1, 2}
    n = 4000
    counts = torch.zeros(6)
    for i in range(n):
        counts[pl.sample_plain(logits, 0.7, 0, 1.0, (i + 0.5) / n)] += 1
    want = torch.zeros(6)
    want[[0, 1, 2, 3, 5]] = torch.softmax(logits[[0, 1, 2, 3, 5]] / 0.7, 0)
    assert float((counts / n - want).abs().max()) < 2e-3


def test_sampling_params_follow_the_reference_defaults():
    p = SamplingParams()
    assert (p.max_tokens, p.temperature, p.top_k, p.top_p, p.seed, p.stop_token_ids) == (32, 0.8, 40, 0.95, None, [])
    assert SamplingParams(max_tokens=0).max_tokens == 1
    assert SamplingParams(temperature=1e-5).greedy and not SamplingParams(temperature=2e-5).greedy
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1)


def test_uniform_numbers():
    us = [uniform(7, i) for i in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 1990
    assert us == [uniform(7, i) for i in range(2000)] and uniform(8, 0) != uniform(7, 0)
    assert abs(sum(us) / len(us) - 0.5) < 0.03
    assert all(float(torch.tensor(u, dtype=torch.float32)) == u for u in us[:50])   # exact in float32
