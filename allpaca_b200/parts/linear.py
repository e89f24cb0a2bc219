"""A weight matrix ``[out, in]`` and the choice of kernel for ``a @ W^T``.

float32 runs on the CUDA cores with 32-bit accumulation (the true 32-bit path);
bfloat16 runs on the tcgen05 tensor cores when the shape allows TMA (rows of a
multiple of 8 elements), else on the CUDA-core kernel.  For few rows the
tensor-core kernel splits K over the CTAs of a thread-block cluster, which add their
partial tiles through distributed shared memory.  Consumers also accept 32-bit partial
sums ``[S, T, N]`` and add them in order (S is 1 for everything produced here).

Reference parity: weights are ``[out, in]`` row-major and ``y = W x`` is ``matmul_nt``
(crates/allpaca-cpu/src/kernels.rs:98-130); no biases on this path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import BuildEnv, Deferred


class Linear:
    def __init__(self, env: BuildEnv, out_features: int, in_features: int):
        self.env = env
        self.out_features = int(out_features)
        self.in_features = int(in_features)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def load(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """``bias`` (``[out]``, optional) is added to the finished sums by a kernel of its own, after
        they were rounded to the output type; nothing on the Llama path has one."""
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"weight {tuple(weight.shape)} is not "
                             f"[{self.out_features}, {self.in_features}]")
        self.weight = weight.contiguous()
        if bias is not None and tuple(bias.shape) != (self.out_features,):
            raise ValueError(f"bias {tuple(bias.shape)} is not [{self.out_features}]")
        self.bias = bias.contiguous() if bias is not None else None

    def uses_tensor_cores(self) -> bool:
        return (self.weight.dtype == torch.bfloat16 and self.in_features % 8 == 0
                and ops.tensor_core_gemm_available())

    # Rows up to which the products of a step take the norm before them as a scale of their result
    # and add into the residual themselves.  Measured on the 8B shape (decode, 4096 keys): a gain of
    # 2 to 5 % of the step up to 16 rows; from 32 rows on the separate norm kernels are faster (a
    # product then has to sum up 128 and more partial sums of squares for each of its many rows).
    FUSED_MAX_ROWS = 16

    def fold_input_scale(self, scale: torch.Tensor) -> None:
        """Multiply ``scale [in]`` (the weight of the norm that produces this product's input) into
        the weight's columns; the sum is formed in 32-bit and rounded once."""
        self.weight = (self.weight.float() * scale.float()[None, :]).to(self.weight.dtype).contiguous()

    def fusable(self) -> bool:
        return self.weight is not None and self.uses_tensor_cores() and self.bias is None

    def residual_rows_ok(self, T: int) -> bool:
        """Whether :meth:`forward_residual` takes ``T`` rows (the K slices of the plan must form a
        cluster of 2, 4 or 8, or be one)."""
        return (self.fusable() and T <= self.FUSED_MAX_ROWS
                and ops.gemm_tc_splits(T, self.out_features, self.in_features) in (1, 2, 4, 8))

    def forward_residual(self, a: torch.Tensor, x: torch.Tensor, buffer_name: str) -> Deferred:
        """``x += a W^T`` in the product's epilogue; returns the updated residual's bfloat16 copy and
        the partial sums of squares of its rows."""
        T, N = a.shape[0], self.out_features
        ws = self.env.workspace
        nsplit = ops.gemm_tc_splits(T, N, self.in_features)
        parts = ops.gemm_tc_residual_parts(N, nsplit)
        xb = ws.get(buffer_name + ".xb", (T, N), torch.bfloat16)
        ss = ws.get(buffer_name + ".ss", (T, parts), torch.float32)
        ops.gemm_tc_residual(a, self.weight, x, xb, ss, nsplit)
        return Deferred(xb, ss, parts)

    def forward(self, a: torch.Tensor, buffer_name: str, kind: str, scale=None) -> torch.Tensor:
        """``a [T, in]`` times the weight.

        ``kind`` says what the consumer takes:
        ``"delta"``   32-bit ``[1, T, out]`` for the residual (consumers take ``[S, T, out]``);
        ``"either"``  ``[T, out]`` in the activation type;
        ``"float32"`` 32-bit ``[T, out]`` (logits).
        ``scale`` (:class:`ops.RowScale`, at most ``FUSED_MAX_ROWS`` rows on the tensor cores): the
        result's rows are scaled in the epilogue.
        """
        T = a.shape[0]
        N = self.out_features
        ws = self.env.workspace
        tc = self.uses_tensor_cores()
        # K slices of the tensor-core kernel add up inside a thread-block cluster, so every
        # kind of consumer gets finished sums; S stays 1
        nsplit = ops.gemm_tc_splits(T, N, self.in_features) if tc else 1
        if kind == "delta":
            out = ws.get(buffer_name, (1, T, N), torch.float32)
            target = out[0]
        else:
            out = ws.get(buffer_name, (T, N), torch.float32 if kind == "float32" else self.env.dtype)
            target = out
        if tc and T > 64 and nsplit > 1:
            # up to 256 rows against few weight tiles: K slices in a cluster, as for decoding
            ops.gemm_tc(a, self.weight, target, nsplit, reduce=True)
        elif tc and ops.gemm_tc_prefers_pair(T, N, self.in_features):
            ops.gemm_tc_pair(a, self.weight, target)
        elif tc and T > 64 and ops.gemm_tc_prefers_persistent(T, N, self.in_features):
            ops.gemm_tc_persistent(a, self.weight, target)
        elif tc and nsplit == 1 and ops.gemm_tc_prefers_dual(T, N, self.in_features):
            ops.gemm_tc_dual(a, self.weight, target)
        elif tc:
            ops.gemm_tc(a, self.weight, target, nsplit, reduce=nsplit > 1, scale=scale)
            scale = None
        else:
            ops.gemm_simt(a, self.weight, target)
        if scale is not None:
            raise ValueError("a scale of the rows is only applied by the tensor-core kernel for few rows")
        if self.bias is not None:
            ops.bias_add(target, self.bias)
        return out

    def forward_gated(self, a: torch.Tensor, buffer_name: str, scale=None) -> Optional[torch.Tensor]:
        """For a weight whose rows alternate gate and up: ``silu(a W_gate^T) * (a W_up^T)`` in one
        kernel, ``[T, out/2]`` in the activation type; None when the shape is not one the fused
        kernel is used for (the caller then multiplies and activates separately)."""
        T = a.shape[0]
        if not self.uses_tensor_cores() or self.out_features % 2 or self.bias is not None:
            return None
        out = self.env.workspace.get(buffer_name, (T, self.out_features // 2), self.env.dtype)
        nsplit = ops.gemm_tc_splits(T, self.out_features, self.in_features)
        if T > 128 and nsplit == 1:
            if scale is not None:
                raise ValueError("a scale of the rows is only applied by the tensor-core kernel for few rows")
            if ops.gemm_tc_prefers_pair(T, self.out_features, self.in_features):
                ops.gemm_tc_pair(a, self.weight, out, pairs=True)
            else:
                ops.gemm_tc_persistent(a, self.weight, out, pairs=True)
        else:
            ops.gemm_tc(a, self.weight, out, nsplit, reduce=nsplit > 1, pairs=True, scale=scale)
        return out
