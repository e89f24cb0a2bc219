"""Settings of the engine around a model: cache geometry, batching limits, dtype.

Role in the reference: the sections of its TOML ``Config`` that this path reads
(crates/allpaca-types/src/config.rs:13-41 with ``validate`` :284-321):
``kv.page_tokens`` (default 128 there), ``prefill.chunk_tokens`` (512, :332-335),
``engine.max_active_requests`` and ``engine.determinism_seed``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .model_config import ConfigError

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
        raise ConfigError(f"dtype {name} is not supported (bfloat16, float32)")
    try:
        return _DTYPES[str(name).lower().replace("torch.", "")]
    except KeyError:
        raise ConfigError(f"dtype {name!r} is not supported (bfloat16, float32)") from None


@dataclass
class EngineConfig:
    dtype: torch.dtype = torch.bfloat16
    page_size: int = 16                     # tokens per cache page (kv.page_tokens)
    num_pages: Optional[int] = None         # pages per cache group; None: from memory
    max_cache_tokens: Optional[int] = None  # alternative to num_pages
    gpu_memory_fraction: float = 0.85       # of free memory, when neither is given
    max_num_seqs: int = 64                  # running requests (engine.max_active_requests)
    max_num_batched_tokens: int = 2048      # rows of one step
    prefill_chunk: int = 512                # largest portion of one prompt in a step
    max_model_len: Optional[int] = None     # None: the model's max_position_embeddings
    seed: int = 0xA110ACA                   # crates/allpaca-core/src/sampling.rs:6
    use_cuda_graphs: bool = True
    device: str = "cuda:0"
    float32_weights: str = "keep"           # matrices stored in 32-bit under a bfloat16 engine: keep | round | refuse

    def validate(self) -> None:
        self.dtype = parse_dtype(self.dtype)
        for k in ("page_size", "max_num_seqs", "max_num_batched_tokens", "prefill_chunk"):
            if int(getattr(self, k)) <= 0:
                raise ConfigError(f"{k} must be positive")
        if self.num_pages is not None and self.num_pages <= 0:
            raise ConfigError("num_pages must be positive")
        if not (0.0 < self.gpu_memory_fraction <= 1.0):
            raise ConfigError("gpu_memory_fraction must be in (0, 1]")
        if self.float32_weights not in ("keep", "round", "refuse"):
            raise ConfigError(f"float32_weights must be keep, round or refuse, not {self.float32_weights!r}")
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ConfigError("max_num_batched_tokens must allow one row per running request "
                              f"({self.max_num_batched_tokens} < {self.max_num_seqs})")
