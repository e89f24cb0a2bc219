"""Command line: ``allpaca generate`` and ``allpaca init-random``.

Option names follow the reference where it has them (``--config``, ``--model``,
``--synthetic``, ``--seed`` of crates/allpaca-server/src/cli.rs:6-73; TOML sections and keys of
allpaca.example.toml: ``[model] path``, ``[engine] max_active_requests, determinism_seed,
target_device``, ``[prefill] chunk_tokens``, ``[kv] page_tokens``, ``[sampling] temperature,
top_k, top_p``).  Precedence as there: compiled defaults < file < command line
(crates/allpaca-types/src/config.rs:98-181).  The reference has no ``generate`` command (it
serves HTTP); this engine works on token ids, so prompts are given as ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from typing import List, Optional, Sequence


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _load_toml(path: Optional[str]) -> dict:
    if path is None:
        path = "allpaca.toml" if os.path.isfile("allpaca.toml") else None
    if path is None:
        return {}
    import tomllib
    with open(path, "rb") as f:
        return tomllib.load(f)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="allpaca", description="allpaca_b200: Llama inference on one B200")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("--config", help="TOML file (sections model, engine, prefill, kv, sampling)")
    g.add_argument("--model", help="folder with config.json and model.safetensors")
    g.add_argument("--synthetic", nargs="?", const="tiny-a", metavar="PRESET",
                   help="random weights of a named shape instead of a checkpoint (default tiny-a)")
    g.add_argument("--seed", type=int, help="seed of random weights and of sampling")
    g.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                   help="one prompt as token ids, comma or space separated (repeatable)")
    g.add_argument("--prompt-file", help="JSON file: a list of token-id lists")
    g.add_argument("--max-tokens", type=int)
    g.add_argument("--temperature", type=float)
    g.add_argument("--top-k", type=int)
    g.add_argument("--top-p", type=float)
    g.add_argument("--stop-token-ids", default="", help="token ids that end a reply")
    g.add_argument("--dtype", choices=["bfloat16", "float32", "auto"], default=None,
                   help="default: what the model folder's config.json names as torch_dtype")
    g.add_argument("--float32-weights", choices=["keep", "round", "refuse"], default="keep",
                   help="matrices stored in 32-bit under --dtype bfloat16: keep them (slow, announced), "
                        "round them to bfloat16 at load, or refuse the checkpoint")
    g.add_argument("--page-tokens", "--page-size", dest="page_tokens", type=int, help="tokens per cache page")
    g.add_argument("--chunk-tokens", "--prefill-chunk", dest="chunk_tokens", type=int,
                   help="largest portion of one prompt per step")
    g.add_argument("--max-active-requests", type=int, help="requests running at a time")
    g.add_argument("--max-cache-tokens", type=int, help="size of the cache pool in tokens")
    g.add_argument("--json", action="store_true", help="one JSON object per reply")

    r = sub.add_parser("init-random", help="write a model folder with random weights")
    r.add_argument("--preset", help="a named shape shipped with the package")
    r.add_argument("--config", help="a config.json to take the sizes from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-std", type=float, default=0.0)
    return p


def _config_dict(preset: Optional[str], config: Optional[str]) -> dict:
    from .config.presets import preset_config
    from .config.model_config import read_config_json
    if preset:
        return preset_config(preset)
    if config:
        return read_config_json(config)
    raise SystemExit("allpaca: give --preset or --config")


def cmd_init_random(args) -> int:
    from .weights.random_model import write_random_model
    write_random_model(args.out, _config_dict(args.preset, args.config), args.seed, args.dtype,
                       std=args.std, norm_std=args.norm_std)
    print(f"wrote {args.out}")
    return 0


def cmd_generate(args) -> int:
    file = _load_toml(args.config)
    sec = lambda name: file.get(name, {}) or {}   # noqa: E731
    pick = lambda cli, *path_default: cli if cli is not None else path_default[0]   # noqa: E731
    model_path = pick(args.model, sec("model").get("path"))
    synthetic = args.synthetic or ("tiny-a" if sec("model").get("synthetic") else None)
    seed = pick(args.seed, sec("engine").get("determinism_seed"))
    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [list(map(int, p)) for p in json.load(f)]
    if not prompts:
        raise SystemExit("allpaca generate: give --prompt-ids or --prompt-file")
    from . import LLM, SamplingParams
    defaults = SamplingParams()
    params = SamplingParams(
        max_tokens=pick(args.max_tokens, defaults.max_tokens),
        temperature=pick(args.temperature, sec("sampling").get("temperature", defaults.temperature)),
        top_k=pick(args.top_k, sec("sampling").get("top_k", defaults.top_k)),
        top_p=pick(args.top_p, sec("sampling").get("top_p", defaults.top_p)),
        seed=seed, stop_token_ids=_ids(args.stop_token_ids))
    tmp = None
    if synthetic and not model_path:
        from .config.presets import preset_config
        from .weights.random_model import write_random_model
        tmp = tempfile.TemporaryDirectory()
        dtype = args.dtype or "bfloat16"
        write_random_model(tmp.name, preset_config(synthetic), seed or 0, dtype)
        model_path = tmp.name
    if not model_path:
        raise SystemExit("allpaca generate: give --model DIR or --synthetic [PRESET]")
    llm = LLM(model=model_path, dtype=args.dtype or "auto", seed=seed, float32_weights=args.float32_weights,
              page_size=pick(args.page_tokens, sec("kv").get("page_tokens", 16)),
              prefill_chunk=pick(args.chunk_tokens, sec("prefill").get("chunk_tokens", 512)),
              max_num_seqs=pick(args.max_active_requests, sec("engine").get("max_active_requests", 64)),
              max_cache_tokens=pick(args.max_cache_tokens, None),
              device=str(sec("engine").get("target_device", "cuda:0")).replace("auto", "cuda:0"))
    for out in llm.generate(prompts, params):
        if args.json:
            print(json.dumps({"token_ids": out.token_ids, "prompt_tokens": out.prompt_tokens,
                              "completion_tokens": out.completion_tokens,
                              "finish_reason": out.finish_reason}))
        else:
            print(" ".join(map(str, out.token_ids)) + f"   [{out.finish_reason}]")
    if tmp is not None:
        tmp.cleanup()
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "init-random":
        return cmd_init_random(args)
    return cmd_generate(args)


if __name__ == "__main__":
    sys.exit(main())
