"""Configurations drawn at random (head sizes from 16 to 256 in steps of 16, groups that do and
do not divide a tile, widths, vocabularies and page sizes that are no power of two) through
the engine in 32-bit and in bfloat16 against the plain implementation: the whole prompt in
one step, then portions beside another request's decoding, then the last tokens one by one."""
import random

import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu


def draw(seed):
    rnd = random.Random(seed)
    hd = rnd.choice([16, 32, 48, 64, 80, 96, 112, 128, 256])
    nkv = rnd.choice([1, 2, 3, 4])
    nh = nkv * rnd.choice([1, 2, 3, 4, 5, 8])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": rnd.choice([1, 2, 3]),
           "hidden_size": 8 * rnd.randrange(8, 40), "num_attention_heads": nh, "num_key_value_heads": nkv,
           "head_dim": hd, "intermediate_size": 8 * rnd.randrange(10, 60),
           "vocab_size": rnd.choice([130, 257, 300, 511, 1000]), "rope_theta": rnd.choice([10000.0, 500000.0]),
           "rms_norm_eps": rnd.choice([1e-5, 1e-6]), "max_position_embeddings": 1024,
           "tie_word_embeddings": rnd.choice([True, False])}
    if rnd.random() < 0.4:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                               "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    return cfg, rnd.choice([4, 8, 16, 32, 64]), rnd.choice([70, 150, 333])


@pytest.mark.parametrize("seed", [57, 62, 26, 84, 47, 9, 35, 65])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(tmp_path, seed, dtype):
    from allpaca_b200 import ops
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    cfg, page, n = draw(seed)
    model = helpers.make_model_folder(str(tmp_path / "m"), cfg, seed, dtype)
    toks = helpers.random_tokens(n, cfg["vocab_size"], seed)
    plain = helpers.plain_logits(model, toks, dtype)
    runner = ModelRunner(model, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=2048, max_num_seqs=4,
                                             max_num_batched_tokens=512))
    want = sorted({0, 1, n // 2, n - 2, n - 1})
    whole = runner.step([BatchEntry("w", toks, want)]).double().cpu().numpy()
    assert np.abs(whole - plain[want]).max() / np.abs(plain[want]).max() < helpers.TOL[dtype], cfg
    runner.finish("w")
    got = {}
    at = 0
    runner.step([BatchEntry("o", toks[:9], [])])
    for k, c in enumerate([n // 3, 2, n - 20 - n // 3 - 2]):
        out = runner.step([BatchEntry("o", toks[9 + k:10 + k], [0]), BatchEntry("p", toks[at:at + c], [c - 1])])
        got[at + c - 1] = out[1].double().cpu().numpy()
        at += c
    while at < n:
        got[at] = runner.step([BatchEntry("p", toks[at:at + 1], [0])])[0].double().cpu().numpy()
        at += 1
    ops.check_kernel_status()
    worst = max(np.abs(v - plain[i]).max() / np.abs(plain[i]).max() for i, v in got.items())
    assert worst < helpers.TOL[dtype], (cfg, page, n)
