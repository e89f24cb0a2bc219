"""The 32-bit path gives a row the same bits whatever else is in the batch, however its
prompt was cut into steps and whichever pages it lies in.

The kernels are written for it: the CUDA-core product sums k in ascending order inside one
thread per output, the norm reduces a row inside one block in a fixed order, and the 32-bit
attention walks a row's keys in chunks that start at the row's first visible position, not at
a portion's edge.  The reference guards the same property of its kernels
(crates/allpaca-cuda/src/lib.rs:5841-5903, crates/allpaca-core/src/model.rs:10851-10863).
bfloat16 is not covered: its kernels are chosen by the size of the batch and differ in
the order of their sums; there the logits agree within rounding (tests/test_replay_gpu.py)."""
import pytest
import torch

import helpers
from helpers import CONFIGS

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_rows_32_bit_logits_do_not_depend_on_batch_or_schedule(tmp_path, name):
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner

    config, seed = CONFIGS[name]
    model = helpers.make_model_folder(str(tmp_path / "m"), config, seed, "float32")
    vocab = config["vocab_size"]
    runner = ModelRunner(model, EngineConfig(dtype="float32", page_size=8, num_pages=64, max_num_seqs=4,
                                             max_num_batched_tokens=256, use_cuda_graphs=False))
    R = helpers.random_tokens(61, vocab, 7)
    others = {k: helpers.random_tokens(n, vocab, 20 + i) for i, (k, n) in enumerate((("x", 33), ("y", 18), ("z", 47)))}
    every = list(range(len(R)))

    # 1. alone and whole
    alone = runner.step([BatchEntry("r", R, every)]).clone()
    runner.finish("r")

    # 2. whole, but inside a mixed step: two other requests are decoding (their prompts ran in
    #    the step before, so the pages R gets are others than in 1), a third brings a portion
    runner.step([BatchEntry("x", others["x"][:-1], []), BatchEntry("y", others["y"][:-1], [])])
    mixed = runner.step([BatchEntry("x", others["x"][-1:], [0]), BatchEntry("y", others["y"][-1:], [0]),
                         BatchEntry("r", R, every), BatchEntry("z", others["z"][:29], [28])])
    assert torch.equal(mixed[2:2 + len(R)], alone), "a row's logits changed with the company it keeps"
    for k in ("r", "x", "y", "z"):
        runner.finish(k)

    # 3. cut into portions of changing size, down to two tokens and single rows, beside another
    #    request that goes on decoding; pages are the ones just given back, in another order
    got = []
    at = 0
    runner.step([BatchEntry("z", others["z"][:20], [])])
    zi = 20
    for n in (2, 7, 1, 16, 3, 1, 1, 25, 5):
        entries = [BatchEntry("r", R[at:at + n], list(range(n)))]
        if zi < len(others["z"]):
            entries.insert(0, BatchEntry("z", others["z"][zi:zi + 1], [0]))
            zi += 1
        out = runner.step(entries)
        got.append(out[out.shape[0] - n:].clone())
        at += n
    assert at == len(R)
    assert torch.equal(torch.cat(got), alone), "a row's logits changed with the way its prompt was cut"
    runner.finish("r"), runner.finish("z")
    runner.cache.check()
