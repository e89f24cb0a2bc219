"""RMSNorm fused with the residual addition that precedes it.

``ss = sum x^2; inv = 1/sqrt(ss/n + eps); out = x * inv * w`` — eps inside the root,
weight multiplied last, no ``+1`` (crates/allpaca-cpu/src/kernels.rs:492-507; CUDA
cuda/src/kernels.cu:1152-1175).  The sum is 32-bit whatever the storage type.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, Norm, WeightSpec, register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """Parameters: ``size`` (width of a row), ``eps``."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("size", "eps")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None
        self._kernel_weight = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.size,), "norm")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()
        self._kernel_weight = self.weight

    def fold(self) -> None:
        """The weight has been multiplied into the product that consumes this norm's output:
        from now on the kernel only divides by the root mean square."""
        self._kernel_weight = torch.ones_like(self.weight)

    @property
    def folded(self) -> bool:
        return self._kernel_weight is not self.weight

    def forward(self, x, out, delta=None, rows=None) -> None:
        ops.add_rmsnorm(x, self._kernel_weight, self.eps, out, delta=delta, rows=rows)
