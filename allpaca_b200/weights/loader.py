"""Weights by tensor name: from safetensors, or random from a configuration and a seed.

Stored types are kept: floating tensors go to the engine's type (bfloat16, or float32 for
the 32-bit path; a tensor stored in 32-bit stays 32-bit), integer tables become int32.
A matrix that stays 32-bit in a bfloat16 engine runs on the slow CUDA-core product: that is
said aloud once per load, and ``float32_weights`` chooses otherwise (``"round"`` them to
bfloat16 at load, or ``"refuse"`` the checkpoint); vectors (norm weights, biases) cost nothing
in 32-bit and always stay.
Every problem of a checkpoint is reported in one error that lists the missing tensors,
the unexpected ones and those of the wrong shape.

Role in the reference: ``TinyModel::from_safetensors``
(crates/allpaca-core/src/model.rs:7904-8044) with lookup by name
(crates/allpaca-safetensors/src/catalog.rs:117-127) and the seeded ``synthetic`` model
(model.rs:5061-5149).  Random weights here follow the distributions the benchmark
configurations name: N(0, std) for matrices, ``1 + N(0, norm_std)`` for norm weights.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from typing import Dict, Mapping, Tuple

import torch

from ..parts import WeightSpec
from .safetensors_io import Checkpoint, write_safetensors


class WeightError(ValueError):
    """A checkpoint that does not fit the model."""


def storage_dtype(stored: torch.dtype, engine: torch.dtype) -> torch.dtype:
    """The type a stored tensor takes on the device."""
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    if stored == torch.float32 or stored == torch.float64:
        return torch.float32
    return engine


def check_names(targets: Mapping[str, Tuple[WeightSpec, object, str]],
                available: Mapping[str, Tuple[int, ...]], ignore_prefixes=()) -> None:
    """Raise one :class:`WeightError` listing everything wrong with the tensor set."""
    missing = [n for n, (ws, _, _) in targets.items() if n not in available and not ws.optional]
    unexpected = [n for n in available if n not in targets
                  and not any(n.startswith(p) for p in ignore_prefixes)]
    wrong = [f"{n}: has {list(available[n])}, expected {list(ws.shape)}"
             for n, (ws, _, _) in targets.items()
             if n in available and tuple(available[n]) != tuple(ws.shape)]
    if missing or unexpected or wrong:
        lines = ["the checkpoint does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightError("\n".join(lines))


FLOAT32_WEIGHT_POLICIES = ("keep", "round", "refuse")


def load_checkpoint(model, path: str, engine_dtype: torch.dtype, device: torch.device,
                    float32_weights: str = "keep") -> None:
    """Read every tensor the model names from a model folder and hand them to the parts.

    ``float32_weights`` says what happens to matrices stored in 32-bit when the engine runs in
    bfloat16: ``"keep"`` them (slow CUDA-core products, announced on standard error),
    ``"round"`` them to bfloat16, or ``"refuse"`` the checkpoint."""
    if float32_weights not in FLOAT32_WEIGHT_POLICIES:
        raise WeightError(f"float32_weights must be one of {FLOAT32_WEIGHT_POLICIES}, not {float32_weights!r}")
    ckpt = Checkpoint(path)
    targets = model.weight_targets()
    wide = []
    # buffers some exporters save beside the weights; they are recomputed from the configuration
    derived = (".rotary_emb.inv_freq",)
    check_names(targets, {n: ckpt.info(n)[1] for n in ckpt.names() if not n.endswith(derived)})
    tensors: Dict[str, torch.Tensor] = {}
    for name in targets:
        if name not in ckpt:
            continue
        t = ckpt.tensor(name)
        want = storage_dtype(t.dtype, engine_dtype)
        if engine_dtype == torch.float32 and t.dtype.is_floating_point:
            want = torch.float32          # the 32-bit path widens 16-bit checkpoints
        elif want == torch.float32 and targets[name][0].role in ("linear", "embedding"):
            wide.append(name)
            if float32_weights == "round":
                want = engine_dtype
        tensors[name] = t.to(device=device, dtype=want, non_blocking=False).contiguous()
    if wide and float32_weights == "refuse":
        raise WeightError(f"{len(wide)} matrices of {path} are stored in 32-bit (first: {wide[0]}) and the engine "
                          f"runs in bfloat16: run it with dtype float32, or let float32_weights round or keep them")
    if wide and float32_weights == "keep":
        print(f"[allpaca_b200] warning: {len(wide)} matrices of {path} are stored in 32-bit (first: {wide[0]}); "
              f"in a bfloat16 engine they stay 32-bit and their products run on the CUDA cores, far slower "
              f"than the tensor cores.  Use dtype float32 for the true 32-bit path, or float32_weights='round' "
              f"to round them to bfloat16 at load.", file=sys.stderr, flush=True)
    model.load_weights(tensors)


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: WeightSpec, seed: int, dtype: torch.dtype,
                  device: torch.device, std: float, norm_std: float) -> torch.Tensor:
    """One tensor drawn from the generator keyed by ``(seed, name)`` on ``device``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, name))
    # always drawn in 32-bit, then rounded: the bfloat16 model is the rounding of the 32-bit one
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    if spec.role == "norm":
        if norm_std > 0:
            t.normal_(0.0, norm_std, generator=gen).add_(1.0)
        else:
            t.fill_(1.0)
    else:
        t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


def random_weights(model, seed: int, dtype: torch.dtype, device: torch.device,
                   std: float = 0.02, norm_std: float = 0.0,
                   tie_word_embeddings: bool = False) -> Dict[str, torch.Tensor]:
    """All tensors of a model in checkpoint names (the head is left out when tied)."""
    out: Dict[str, torch.Tensor] = {}
    for name, (spec, _, local) in model.weight_targets().items():
        if local == "head" and tie_word_embeddings:
            continue
        out[name] = random_tensor(name, spec, seed, dtype, device, std, norm_std)
    return out


def write_model_folder(path: str, config: Mapping, tensors: Mapping[str, torch.Tensor]) -> None:
    """``config.json`` and ``model.safetensors`` of a model folder."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config), f, indent=1, sort_keys=True)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, {"format": "pt"})
