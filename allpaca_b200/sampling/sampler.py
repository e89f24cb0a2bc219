"""Chooses next tokens on the GPU from the logits of a step.

All rows go through one kernel launch: arg-max alone when every row is greedy, else the
sampling kernel, which is greedy per row where the row's temperature is ``<= 1e-5``.
Only the chosen token ids come back to the host (4 bytes a row), not the logits.

Role in the reference: ``sample`` on the CPU over logits copied to the host
(crates/allpaca-core/src/sampling.rs:69-82, crates/allpaca-core/src/engine.rs:7180).
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device: torch.device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        self._host = torch.empty((4, max_rows), dtype=torch.float32, pin_memory=True)
        self._dev = torch.empty((4, max_rows), dtype=torch.float32, device=device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               uniforms: Sequence[float]) -> List[int]:
        """One token per row of ``logits [R, V]``."""
        R = logits.shape[0]
        if R == 0:
            return []
        if R > self.max_rows:
            raise ValueError(f"{R} rows exceed the sampler's {self.max_rows}")
        out = self._out[:R]
        if all(p.greedy for p in params):
            ops.argmax(logits, out)
        else:
            h = self._host.numpy()
            h[0, :R] = [p.temperature for p in params]
            h[1, :R].view(np.int32)[:] = [p.top_k for p in params]
            h[2, :R] = [p.top_p for p in params]
            h[3, :R] = list(uniforms)
            self._dev[:, :R].copy_(self._host[:, :R], non_blocking=True)
            ops.sample(logits, self._dev[0, :R], self._dev[1, :R].view(torch.int32),
                       self._dev[2, :R], self._dev[3, :R], out)
        self._out_host[:R].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:R].tolist()
