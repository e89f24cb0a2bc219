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
