"""A weight matrix ``[out, in]`` and the choice of kernel for ``a @ W^T``.

float32 runs on the CUDA cores with 32-bit accumulation (the true 32-bit path);
bfloat16 runs on the tcgen05 tensor cores when the shape allows TMA (rows of a
multiple of 8 elements), else on the CUDA-core kernel.  For few rows the
tensor-core kernel splits K over several thread blocks and returns 32-bit partial
sums ``[S, T, N]``, which every consumer adds in order.

Reference parity: weights are ``[out, in]`` row-major and ``y = W x`` is ``matmul_nt``
(crates/allpaca-cpu/src/kernels.rs:98-130); no biases on this path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import BuildEnv


class Linear:
    def __init__(self, env: BuildEnv, out_features: int, in_features: int):
        self.env = env
        self.out_features = int(out_features)
        self.in_features = int(in_features)
        self.weight: Optional[torch.Tensor] = None

    def load(self, weight: torch.Tensor) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weight {tuple(weight.shape)} is not "
                             f"[{self.out_features}, {self.in_features}]")
        self.weight = weight.contiguous()

    def uses_tensor_cores(self) -> bool:
        return (self.weight.dtype == torch.bfloat16 and self.in_features % 8 == 0
                and ops.tensor_core_gemm_available())

    def forward(self, a: torch.Tensor, buffer_name: str, kind: str) -> torch.Tensor:
        """``a [T, in]`` times the weight.

        ``kind`` says what the consumer takes:
        ``"delta"``   32-bit partial sums ``[S, T, out]`` (S may be 1), for the residual;
        ``"either"``  ``[T, out]`` in the activation type, or ``[S, T, out]`` partial sums
                      when the kernel chose to split K;
        ``"float32"`` 32-bit ``[T, out]`` (logits).
        """
        T = a.shape[0]
        N = self.out_features
        ws = self.env.workspace
        tc = self.uses_tensor_cores()
        nsplit = ops.gemm_tc_splits(T, N, self.in_features) if (tc and kind != "float32") else 1
        if kind == "delta" or (kind == "either" and nsplit > 1):
            out = ws.get(buffer_name, (nsplit, T, N), torch.float32)
            if tc:
                ops.gemm_tc(a, self.weight, out if nsplit > 1 else out[0], nsplit)
            else:
                ops.gemm_simt(a, self.weight, out[0])
            return out
        out = ws.get(buffer_name, (T, N), torch.float32 if kind == "float32" else self.env.dtype)
        if tc:
            ops.gemm_tc(a, self.weight, out, 1)
        else:
            ops.gemm_simt(a, self.weight, out)
        return out
