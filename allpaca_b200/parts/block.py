"""The pre-norm arrangement of a decoder layer.

``x -> norm -> mixer -> +x -> norm -> feed-forward -> +x``
(crates/allpaca-core/src/model.rs:8447-8696).  The residual ``x`` is 32-bit; each addition
is performed inside the norm that follows it, which reads the pending partial sums, so the
block hands its last addition to whoever runs next.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import Block, BuildEnv, Deferred, LayerCache, Part, build, register
from .norm import RMSNorm


@register("block", "prenorm")
class PreNormBlock(Block):
    """Parameters: ``hidden_size`` and four :class:`PartSpec`: ``mixer``, ``feed_forward``,
    ``mixer_norm``, ``feed_forward_norm``; and the weight-name prefixes ``mixer_prefix``,
    ``feed_forward_prefix``, ``mixer_norm_prefix``, ``feed_forward_norm_prefix``."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "mixer", "feed_forward", "mixer_norm", "feed_forward_norm")
        self.hidden = int(params["hidden_size"])
        self.mixer = build("mixer", params["mixer"], env)
        self.feed_forward = build("feed_forward", params["feed_forward"], env)
        self.mixer_norm = build("norm", params["mixer_norm"], env)
        self.feed_forward_norm = build("norm", params["feed_forward_norm"], env)
        self._prefixes = {
            params.get("mixer_prefix", "mixer."): self.mixer,
            params.get("feed_forward_prefix", "feed_forward."): self.feed_forward,
            params.get("mixer_norm_prefix", "mixer_norm."): self.mixer_norm,
            params.get("feed_forward_norm_prefix", "feed_forward_norm."): self.feed_forward_norm,
        }

        self.fused = False

    def sub_parts(self) -> Dict[str, Part]:
        return dict(self._prefixes)

    def finalize(self) -> None:
        """In bfloat16, where both norms are RMSNorm and mixer and feed-forward can take it: the
        norms' weights are multiplied into the products that follow them.  A step of few rows then
        runs without norm kernels (the products scale their result rows by the root mean square,
        which the product before them summed up while it added into the residual); a step of many
        rows runs the norm kernels as before, without their weights."""
        if self.env.dtype != torch.bfloat16:
            return
        if not (type(self.mixer_norm) is RMSNorm and type(self.feed_forward_norm) is RMSNorm):
            return
        if self.mixer_norm.folded or self.feed_forward_norm.folded:
            return                      # done before (weights are folded once per load)
        self.fused = False
        can = [getattr(part, "can_fold_input_norm", lambda: False)() for part in (self.mixer, self.feed_forward)]
        if not all(can):
            return
        self.mixer.fold_input_norm(self.mixer_norm.weight)
        self.feed_forward.fold_input_norm(self.feed_forward_norm.weight)
        self.mixer_norm.fold()
        self.feed_forward_norm.fold()
        self.fused = True

    def forward(self, x: torch.Tensor, delta, step, cache: LayerCache):
        T = x.shape[0]
        h = self.env.workspace.get("block.normed", (T, self.hidden), self.env.dtype)
        if self.fused and self.mixer.fused_rows_ok(T) and self.feed_forward.fused_rows_ok(T):
            if isinstance(delta, Deferred):
                inp, scale = delta.xb, ops.RowScale(delta.ss, delta.parts, self.hidden, self.mixer_norm.eps)
            else:
                self.mixer_norm.forward(x, h, delta=delta)
                inp, scale = h, None
            d = self.mixer.forward_fused(inp, scale, x, step, cache)
            scale = ops.RowScale(d.ss, d.parts, self.hidden, self.feed_forward_norm.eps)
            return self.feed_forward.forward_fused(d.xb, scale, x, step)
        if isinstance(delta, Deferred):
            delta = None                 # the block before has added into the residual itself
        self.mixer_norm.forward(x, h, delta=delta)
        delta = self.mixer.forward(h, step, cache)
        self.feed_forward_norm.forward(x, h, delta=delta)
        return self.feed_forward.forward(h, step)
