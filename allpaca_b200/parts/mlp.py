"""SwiGLU feed-forward: ``down( silu(gate h) * (up h) )``.

``silu(z) = z / (1 + exp(-z))`` (crates/allpaca-cpu/src/kernels.rs:869-871); gate and up
are separate tensors in the checkpoint (crates/allpaca-core/src/model.rs:5664-5705) and one
matrix here whose rows alternate gate, up, gate, up ...: one product yields ``[T, 2I]`` with
each (gate, up) pair side by side.  On the tensor cores row 2i and 2i+1 of the weight are
neighbouring lanes of the accumulator, so for many rows the product's epilogue applies the
activation itself; for few rows a small kernel reads the pairs.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, FeedForward, WeightSpec, register
from .linear import Linear


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``bias`` (False: no biases, as on the
    Llama path)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "intermediate_size")
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.bias = bool(params.get("bias", False))
        self.gate_up = Linear(env, 2 * self.inter, self.hidden)
        self.down = Linear(env, self.hidden, self.inter)

    def weights(self) -> Dict[str, WeightSpec]:
        w = {"gate_proj.weight": WeightSpec((self.inter, self.hidden)),
             "up_proj.weight": WeightSpec((self.inter, self.hidden)),
             "down_proj.weight": WeightSpec((self.hidden, self.inter))}
        if self.bias:
            w.update({"gate_proj.bias": WeightSpec((self.inter,), "bias"),
                      "up_proj.bias": WeightSpec((self.inter,), "bias"),
                      "down_proj.bias": WeightSpec((self.hidden,), "bias")})
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        gu_bias = torch.stack([tensors["gate_proj.bias"], tensors["up_proj.bias"]], dim=1).reshape(-1) \
            if self.bias else None
        self.gate_up.load(torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden), gu_bias)
        self.down.load(tensors["down_proj.weight"], tensors["down_proj.bias"] if self.bias else None)

    def can_fold_input_norm(self) -> bool:
        return self.gate_up.fusable() and self.down.fusable()

    def fold_input_norm(self, weight: torch.Tensor) -> None:
        """Multiply the weight of the norm before this feed-forward into its first product."""
        self.gate_up.fold_input_scale(weight)

    def fused_rows_ok(self, T: int) -> bool:
        return T <= Linear.FUSED_MAX_ROWS and self.down.residual_rows_ok(T)

    def forward_fused(self, h: torch.Tensor, scale, x: torch.Tensor, step):
        """For few rows: ``h`` with ``scale`` (an ``ops.RowScale``) stands for the normed input;
        the down projection adds into ``x`` itself.  Returns a :class:`Deferred`."""
        act = self.gate_up.forward_gated(h, "ffn.act", scale=scale)
        return self.down.forward_residual(act, x, "ffn")

    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        T = h.shape[0]
        act = self.gate_up.forward_gated(h, "ffn.act")        # one kernel when there are many rows
        if act is None:
            gu = self.gate_up.forward(h, "ffn.gate_up", "either")
            act = self.env.workspace.get("ffn.act", (T, self.inter), self.env.dtype)
            ops.swiglu(gu, act, pairs=True)
        return self.down.forward(act, "ffn.down", "delta")
