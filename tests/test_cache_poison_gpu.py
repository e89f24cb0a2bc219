"""A page that comes back from another request may hold anything, NaN and infinity included.

The attention kernels load whole pages and weigh what lies behind a row's position with a
probability of exactly zero; ``0 x NaN`` would poison the row.  The engine therefore clears
the unwritten tail of a page when the page gets its first token (the store of keys and
values does it, ``csrc/elementwise.cu``).  Here every page of the pool is filled with NaN
(or infinity) before requests run: whole prompts, portions, single decoded tokens and
a request that takes over the pages another one just gave back must all give the plain
logits, in 32-bit and in bfloat16 (where the kernels that load whole pages by TMA run)."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

# head size 64, so that the TMA-fed decode attention and the tcgen05 prompt attention are the
# ones that run in bfloat16
CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 192, "vocab_size": 311, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 512, "tie_word_embeddings": False,
}


@pytest.mark.parametrize("junk", [float("nan"), float("inf")])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_full_of_junk_do_not_reach_the_logits(tmp_path, dtype, junk):
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner

    model = helpers.make_model_folder(str(tmp_path / "m"), CONFIG, 4, dtype)
    runner = ModelRunner(model, EngineConfig(dtype=dtype, page_size=16, num_pages=24, max_num_seqs=3,
                                             max_num_batched_tokens=256))
    for storage in runner.storages:
        storage.pages.fill_(junk)
    a = helpers.random_tokens(150, CONFIG["vocab_size"], 1)
    b = helpers.random_tokens(101, CONFIG["vocab_size"], 2)
    plain = {"a": helpers.plain_logits(model, a, dtype), "b": helpers.plain_logits(model, b, dtype)}
    tol = helpers.TOL[dtype]

    def check(logits, rid, positions, what):
        got = logits.double().cpu().numpy()
        assert torch.isfinite(logits).all(), f"{what}: non-finite logits"
        for i, pos in enumerate(positions):
            ref = plain[rid][pos]
            err = abs(got[i] - ref).max() / abs(ref).max()
            assert err <= tol, (what, pos, err)

    # a: 70 tokens at once (the last page is filled to 6 of 16 slots), then a portion of 37 that
    # ends inside a page, then single tokens across a page's edge
    check(runner.step([BatchEntry("a", a[:70], [0, 33, 69])]), "a", [0, 33, 69], "first portion")
    check(runner.step([BatchEntry("a", a[70:107], [0, 36])]), "a", [70, 106], "second portion")
    for i in range(107, 131):
        check(runner.step([BatchEntry("a", a[i:i + 1], [0])]), "a", [i], "decoding")
    # junk again in every page a does not hold, then b starts beside a's decoding
    held = set(runner.cache.block_table("a", 0))
    for storage in runner.storages:
        for page in range(storage.pages.shape[1]):
            if page not in held:
                storage.pages[:, page].fill_(junk)
    out = runner.step([BatchEntry("a", a[131:132], [0]), BatchEntry("b", b[:66], [65])])
    check(out[:1], "a", [131], "decoding beside a new request")
    check(out[1:], "b", [65], "new request on junk pages")
    runner.finish("a")
    # b grows into the pages a gave back (their contents: a's keys, which are not b's)
    for storage in runner.storages:
        for page in held:
            storage.pages[:, page].fill_(junk)
    check(runner.step([BatchEntry("b", b[66:100], [0, 33])]), "b", [66, 99], "portion on pages given back")
    check(runner.step([BatchEntry("b", b[100:101], [0])]), "b", [100], "last token")
    runner.finish("b")
    runner.cache.check()
