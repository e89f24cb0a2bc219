"""Rotary position embedding with optional llama3 frequency scaling.

``freq_i = theta^(-i/half)``, angle ``= pos * freq_i``, pair ``(a, b) -> (a cos - b sin,
a sin + b cos)`` (crates/allpaca-cpu/src/kernels.rs:510-527).  Checkpoints in the Hugging
Face layout pair element ``i`` with ``i + half`` (crates/allpaca-core/src/model.rs:196-199,
:7937; crates/allpaca-cpu/src/kernels.rs:676-682); checkpoints whose Q/K rows were permuted
by a converter pair ``2i`` with ``2i+1`` (model.rs:3215-3227).  Both are a parameter here.

The llama3 scaling is not in the reference (its config has no field for it,
model.rs:181-274).  With ``factor f``, ``low_freq_factor lo``, ``high_freq_factor hi`` and
``original_max_position_embeddings n0``: a pair whose wavelength ``2 pi / freq`` is below
``n0/hi`` keeps its frequency, above ``n0/lo`` it is divided by ``f``, and in between the two
are blended with weight ``s = (n0/wavelength - lo) / (hi - lo)``.

The table of frequencies is computed once in float64 and kept in float32; the angle is a
32-bit product, and its cosine and sine are computed once per step for all layers.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from .. import ops
from .base import BuildEnv, PartError, PositionEncoding, register

PAIRING = {"half": 0, "adjacent": 1}


def inverse_frequencies(head_dim: int, theta: float, scaling: Optional[Mapping]) -> torch.Tensor:
    """float64 ``[head_dim/2]`` rotation frequencies after scaling."""
    half = head_dim // 2
    freqs = []
    for i in range(half):
        f = float(theta) ** (-(i / half))
        if scaling is not None:
            factor = float(scaling["factor"])
            lo = float(scaling["low_freq_factor"])
            hi = float(scaling["high_freq_factor"])
            n0 = float(scaling["original_max_position_embeddings"])
            wavelength = 2.0 * math.pi / f
            if wavelength > n0 / lo:
                f = f / factor
            elif wavelength >= n0 / hi:
                s = (n0 / wavelength - lo) / (hi - lo)
                f = (1.0 - s) * f / factor + s * f
        freqs.append(f)
    return torch.tensor(freqs, dtype=torch.float64)


@register("position", "rope")
class RotaryEmbedding(PositionEncoding):
    """Parameters: ``head_dim``, ``theta``, ``scaling`` (mapping or None), ``pairing``
    (``"half"`` or ``"adjacent"``)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("head_dim", "theta")
        self.head_dim = int(params["head_dim"])
        if self.head_dim % 2:
            raise PartError(f"rotary head_dim {self.head_dim} must be even")
        pairing = params.get("pairing", "half")
        if pairing not in PAIRING:
            raise PartError(f"unknown rotary pairing {pairing!r} (known: {', '.join(PAIRING)})")
        self.pairing = PAIRING[pairing]
        scaling = params.get("scaling")
        if scaling is not None and scaling.get("rope_type", "llama3") != "llama3":
            raise PartError(f"unknown rope scaling {scaling.get('rope_type')!r}")
        self.inv_freq = inverse_frequencies(self.head_dim, float(params["theta"]), scaling) \
            .to(torch.float32).to(env.device)

        self._key = ("rope", self.head_dim, float(params["theta"]), self.pairing,
                     tuple(sorted(scaling.items())) if scaling else None)

    def rotation_for(self, step):
        """``([T, head_dim/2, 2] cos/sin of this step's positions, pairing)``; layers with the
        same rotation share one table per step."""
        table = step.shared.get(self._key)
        if table is None:
            T = step.num_tokens
            table = self.env.workspace.get(f"rope.table.{len(step.shared)}",
                                           (T, self.head_dim // 2, 2), torch.float32)
            ops.rope_table(step.positions, self.inv_freq, table)
            step.shared[self._key] = table
        return table, self.pairing
