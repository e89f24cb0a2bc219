"""Without a CUDA device the engine refuses to run instead of falling back to the CPU."""
import pytest
import torch

from allpaca_b200.config import EngineConfig


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_no_cpu_fallback(tmp_path):
    import helpers
    from allpaca_b200.engine.runner import ModelRunner
    from allpaca_b200.ops import library
    cfg, seed = helpers.CONFIGS["A"]
    model = helpers.make_model_folder(str(tmp_path / "m"), cfg, seed)
    with pytest.raises(RuntimeError, match="CUDA"):
        ModelRunner(model, EngineConfig(dtype="float32"))
    with pytest.raises(library.KernelError, match="no CPU implementation"):
        library._require_cuda()


def test_trace_run_arguments():
    from allpaca_b200.engine import replay
    args = replay.parse_args(["--model", "m", "--dtype", "float32", "--out", "o", "--max-tokens", "256"])
    assert (args.model, args.dtype, args.out, args.max_tokens) == ("m", "float32", "o", 256)
    with pytest.raises(SystemExit):
        replay.parse_args(["--model", "m", "--dtype", "float16", "--out", "o", "--max-tokens", "1"])


def test_command_line_parser():
    from allpaca_b200.cli import build_parser
    a = build_parser().parse_args(["generate", "--synthetic", "--seed", "3", "--prompt-ids", "1,2", "--max-tokens", "4"])
    assert a.synthetic == "tiny-a" and a.seed == 3 and a.prompt_ids == ["1,2"]
    b = build_parser().parse_args(["init-random", "--preset", "tiny-b", "--out", "x"])
    assert b.preset == "tiny-b" and b.dtype == "bfloat16"


def test_plan_of_key_slices_for_decoding():
    """The number of key slices of the decode attention: one slice where the batch fills the
    GPU by itself, more for few sequences, cluster sizes preferred to counts that need a second
    kernel, and 16 (a cluster only few of which find room) for up to 8 clusters alone."""
    from allpaca_b200.ops import decode_splits
    tma = dict(slots=296, cluster_sizes=(2, 4, 8, 16))
    assert decode_splits(64, 32, 8, 4096, **tma) == 1
    assert decode_splits(128, 32, 8, 2048, **tma) == 1 and decode_splits(80, 32, 8, 2048, **tma) == 1
    # sequences of unequal length: the longest sets the slowest CTA's time, so it is cut finer
    assert decode_splits(8, 32, 8, 32768, **tma) == 4 and decode_splits(8, 32, 8, 32768, mean_context=4500, **tma) == 16
    assert decode_splits(128, 32, 8, 16384, **tma) == 1 and decode_splits(128, 32, 8, 16384, mean_context=600, **tma) == 4
    assert decode_splits(8, 32, 8, 4096, mean_context=3500, **tma) == decode_splits(8, 32, 8, 4096, **tma)
    assert decode_splits(8, 32, 8, 4096, **tma) == 4
    assert decode_splits(1, 32, 8, 4096, **tma) == 8
    assert decode_splits(1, 32, 8, 8192, **tma) == 16
    assert decode_splits(2, 32, 8, 8192, **tma) == 8           # 16 clusters of 16 would not find room
    assert decode_splits(1, 32, 8, 8192, slots=296, cluster_sizes=(2, 4, 8)) == 8
    for rows in (1, 3, 8, 40):
        for ctx in (1, 63, 64, 65, 1000, 20000, 131072):
            for window in (0, 100):
                n = decode_splits(rows, 32, 8, ctx, window, **tma)
                keys = min(ctx, window) if window else ctx
                assert 1 <= n <= max(1, -(-keys // 64))          # never more slices than tiles of 64 keys
    assert decode_splits(1, 8, 8, 300, window=0, **tma) == decode_splits(1, 8, 8, 100000, window=300, **tma)
