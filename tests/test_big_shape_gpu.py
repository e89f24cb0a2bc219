"""Two layers of the Llama-3.1-8B shape in true 32-bit against the plain implementation, whole
and cut into portions; and bfloat16 on the same weights (the sizes the benchmark runs)."""
import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("two_query_tiles,page", [(False, 16), (True, 16), (False, 128)])
def test_two_layers_of_the_8b_shape(tmp_path, monkeypatch, two_query_tiles, page):
    """``two_query_tiles``: the prompt attention with two query tiles to a CTA, which the engine
    otherwise keeps for longer portions, takes every portion of 64 rows or more.  ``page``: 128
    tokens to a page (two key tiles of the decode kernel, one of the prompt kernel's)."""
    from allpaca_b200 import ops
    if two_query_tiles:
        monkeypatch.setattr(ops, "WIDE_ATTENTION_MIN_CTAS", 1)
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.config.presets import preset_config
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    from allpaca_b200.parts import BuildEnv, Workspace
    from allpaca_b200.weights.random_model import random_model_on_device

    raw = preset_config("llama-3.1-8b")
    raw["num_hidden_layers"] = 2
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, raw["vocab_size"], (150,), generator=g).tolist()
    want_rows = [0, 1, 63, 64, 127, 128, 149]
    w = None
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        env = BuildEnv(dtype, dev, Workspace(dev), page_size=page, max_seqs=2)
        cfg, model = random_model_on_device(raw, 2, env)
        if w is None:
            # weights are drawn on the GPU in 32-bit (bfloat16 is their rounding): the plain
            # implementation gets the same ones
            w = {}
            for block, prefix in zip(model.blocks, model.spec.layer_prefixes):
                qkv = block.mixer.qkv.weight
                Q, KV = cfg.q_size, cfg.kv_size
                w[prefix + "self_attn.q_proj.weight"] = qkv[:Q]
                w[prefix + "self_attn.k_proj.weight"] = qkv[Q:Q + KV]
                w[prefix + "self_attn.v_proj.weight"] = qkv[Q + KV:]
                w[prefix + "self_attn.o_proj.weight"] = block.mixer.o.weight
                gu = block.feed_forward.gate_up.weight
                w[prefix + "mlp.gate_proj.weight"] = gu[0::2]      # gate and up rows alternate
                w[prefix + "mlp.up_proj.weight"] = gu[1::2]
                w[prefix + "mlp.down_proj.weight"] = block.feed_forward.down.weight
                w[prefix + "input_layernorm.weight"] = block.mixer_norm.weight
                w[prefix + "post_attention_layernorm.weight"] = block.feed_forward_norm.weight
            w["model.embed_tokens.weight"] = model.embedding
            w["lm_head.weight"] = model.head.weight
            w["model.norm.weight"] = model.final_norm.weight
            w = {k: v.cpu() for k, v in w.items()}
        if dtype == torch.float32:
            plain = plain_llama.llama_forward(raw, w, tokens, torch.float32)[want_rows].double()
        else:
            plain = plain_llama.llama_forward(raw, {k: v.bfloat16() for k, v in w.items()}, tokens,
                                              torch.float32, round_to=torch.bfloat16)[want_rows].double()
        runner = ModelRunner(None, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=512, max_num_seqs=2,
                                                max_num_batched_tokens=256, use_cuda_graphs=False), model=model)
        whole = runner.step([BatchEntry("w", tokens, want_rows)]).double().cpu()
        err = float((whole - plain).abs().max() / plain.abs().max())
        assert err < tol, (dtype, "whole", err)
        runner.finish("w")
        # portions 64 + 1 + 63 + 22 beside a second request decoding
        got = []
        at = 0
        for n in (64, 1, 63, 22):
            want = [r - at for r in want_rows if at <= r < at + n]
            entries = [BatchEntry("p", tokens[at:at + n], want)]
            if at > 0:
                entries.append(BatchEntry("other", tokens[at:at + 1], []))
            else:
                entries.append(BatchEntry("other", tokens[:9], []))
            out = runner.step(entries)
            got.append(out[:len(want)].double().cpu())
            at += n
        err = float((torch.cat(got) - plain).abs().max() / plain.abs().max())
        assert err < tol, (dtype, "portions", err)
        del runner, model
        torch.cuda.empty_cache()


# ---------------------------------------------------------------------------
# the same shape through bin/trace_run, in all four ways of cutting and batching
# ---------------------------------------------------------------------------
BIG_LENGTHS = [72, 150, 320]


@pytest.fixture(scope="module")
def big_model(tmp_path_factory):
    """Two layers of the Llama-3.1-8B shape as model folders (float32, and its bfloat16
    rounding), with the requests and what the plain implementation says about them."""
    import helpers
    from allpaca_b200.config.presets import preset_config
    from allpaca_b200.weights.loader import write_model_folder
    raw = preset_config("llama-3.1-8b")
    raw["num_hidden_layers"] = 2
    raw["max_position_embeddings"] = 512
    root = tmp_path_factory.mktemp("big")
    d32 = helpers.make_model_folder(str(root / "f32"), raw, 2, "float32")
    w = helpers.load_weights(d32)
    d16 = str(root / "bf16")
    write_model_folder(d16, dict(helpers.load_config(d32), torch_dtype="bfloat16"),
                       {k: v.to(torch.bfloat16) for k, v in w.items()})
    requests = {str(i): helpers.random_tokens(n, raw["vocab_size"], 500 + i) for i, n in enumerate(BIG_LENGTHS)}
    return {"config": raw, "float32": d32, "bfloat16": d16, "weights": w, "requests": requests}


@pytest.mark.parametrize("dtype,two_query_tiles", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_two_layers_of_the_8b_shape_replayed_in_every_mode(tmp_path, big_model, dtype, two_query_tiles):
    """Whole; the last 32 tokens one by one; portions of changing size down to two tokens; mixed
    with up to four live requests on a pool so small that pages are used again.  At this shape
    the bfloat16 run is the one place where the tcgen05 products and the tcgen05 attention
    (with ``two_query_tiles`` the kernel with two query tiles to a CTA for every portion of 64
    rows or more) are compared with the plain implementation end to end."""
    import os
    import numpy as np
    import helpers
    from test_replay_gpu import build_trace
    tb, alias, peak = build_trace(big_model["requests"], dense=False)
    env = dict(os.environ)
    if two_query_tiles:
        env["ALLPACA_WIDE_ATTENTION_MIN_CTAS"] = "1"
    outputs = helpers.run_trace(big_model[dtype], dtype, str(tmp_path / "out"), tb.steps, peak, env=env,
                                timeout=1500)
    # the plain logits of the rows the trace asks for, per request
    wanted = {}
    for k, rows in tb.rows.items():
        for rid, pos in rows:
            wanted.setdefault(alias[rid], set()).add(pos)
    w = big_model["weights"]
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    reference = {}
    for r, toks in big_model["requests"].items():
        rows = sorted(wanted[r])
        out = plain_llama.llama_forward(big_model["config"], w, toks, torch.float32,
                                        round_to=torch.bfloat16 if dtype == "bfloat16" else None, rows=rows)
        full = {pos: out[i].double().numpy() for i, pos in enumerate(rows)}
        reference[r] = full
    helpers.compare(outputs, tb, {rid: reference[r] for rid, r in alias.items()}, helpers.TOL[dtype],
                    f"8B shape, 2 layers, {dtype}{', two query tiles' if two_query_tiles else ''}")
