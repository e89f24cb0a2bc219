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


class Pending:
    """Tokens chosen by a launched sampling kernel: on the device at once (``device``, int32),
    on the host once :meth:`Sampler.fetch` has waited for the copy."""

    def __init__(self, device: torch.Tensor, host: torch.Tensor, event: torch.cuda.Event, rows: int):
        self.device, self.host, self.event, self.rows = device, host, event, rows


class Sampler:
    def __init__(self, device: torch.device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        self._host = torch.empty((4, max_rows), dtype=torch.float32, pin_memory=True)
        self._dev = torch.empty((4, max_rows), dtype=torch.float32, device=device)
        # two sets of result buffers: the step after this one may read the device tokens while
        # the next launch writes the other set
        self._out = [torch.empty(max_rows, dtype=torch.int32, device=device) for _ in range(2)]
        self._out_host = [torch.empty(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._params_copied = torch.cuda.Event()
        self._params_copied.record()
        self._turn = 0

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               uniforms: Sequence[float]) -> Pending:
        """Choose one token per row of ``logits [R, V]`` on the GPU and start their copy to the
        host; nothing here waits for the GPU."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows exceed the sampler's {self.max_rows}")
        self._turn ^= 1
        out, host, event = self._out[self._turn][:R], self._out_host[self._turn][:R], self._events[self._turn]
        if R == 0:
            event.record()
            return Pending(out, host, event, 0)
        if all(p.greedy for p in params):
            ops.argmax(logits, out)
        else:
            self._params_copied.synchronize()        # the pinned parameters of the launch before are on the device
            h = self._host.numpy()
            h[0, :R] = [p.temperature for p in params]
            h[1, :R].view(np.int32)[:] = [p.top_k for p in params]
            h[2, :R] = [p.top_p for p in params]
            h[3, :R] = list(uniforms)
            self._dev[:, :R].copy_(self._host[:, :R], non_blocking=True)
            self._params_copied.record()
            ops.sample(logits, self._dev[0, :R], self._dev[1, :R].view(torch.int32),
                       self._dev[2, :R], self._dev[3, :R], out)
        host.copy_(out, non_blocking=True)
        event.record()
        return Pending(out, host, event, R)

    def fetch(self, pending: Pending) -> List[int]:
        """The tokens of a launch, once they have arrived."""
        pending.event.synchronize()
        return pending.host[:pending.rows].tolist()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               uniforms: Sequence[float]) -> List[int]:
        """One token per row of ``logits [R, V]``."""
        return self.fetch(self.launch(logits, params, uniforms))
