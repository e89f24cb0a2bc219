"""Random-weights mode: a model folder, or a ready model on the device, from a
configuration and a seed.

Matrices are N(0, std), norm weights ``1 + N(0, norm_std)`` (1 exactly for ``norm_std`` 0),
each tensor drawn from a generator keyed by ``(seed, tensor name)``.  Role in the reference:
``TinyModel::synthetic(cfg, seed, name)`` (crates/allpaca-core/src/model.rs:5061-5149).
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.engine_config import parse_dtype
from ..models import DecoderModel, resolve
from ..parts import BuildEnv, Workspace
from .loader import random_weights, write_model_folder


def _model_for(config: Mapping, dtype: torch.dtype, device: torch.device):
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    env = BuildEnv(dtype=dtype, device=device, workspace=Workspace(device))
    return cfg, DecoderModel(arch.spec_builder(cfg), env), env


def write_random_model(path: str, config: Mapping, seed: int, dtype="float32",
                       std: float = 0.02, norm_std: float = 0.0) -> None:
    """Write ``config.json`` and ``model.safetensors`` of a randomly initialised model."""
    dt = parse_dtype(dtype)
    cfg, model, _ = _model_for(config, dt, torch.device("cpu"))
    tensors = random_weights(model, seed, dt, torch.device("cpu"), std, norm_std,
                             tie_word_embeddings=cfg.tie_word_embeddings)
    out = dict(config)
    out["torch_dtype"] = "float32" if dt == torch.float32 else "bfloat16"
    write_model_folder(path, out, tensors)


def random_model_on_device(config: Mapping, seed: int, env: BuildEnv, std: float = 0.02,
                           norm_std: float = 0.0):
    """(typed config, model with random weights drawn on the device) — no files involved."""
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    model = DecoderModel(arch.spec_builder(cfg), env)
    tensors = random_weights(model, seed, env.dtype, env.device, std, norm_std,
                             tie_word_embeddings=cfg.tie_word_embeddings)
    model.load_weights(tensors)
    return cfg, model
