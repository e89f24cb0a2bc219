"""The pre-norm arrangement of a decoder layer.

``x -> norm -> mixer -> +x -> norm -> feed-forward -> +x``
(crates/allpaca-core/src/model.rs:8447-8696).  The residual ``x`` is 32-bit; each addition
is performed inside the norm that follows it, which reads the pending partial sums, so the
block hands its last addition to whoever runs next.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import Block, BuildEnv, LayerCache, Part, build, register


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

    def sub_parts(self) -> Dict[str, Part]:
        return dict(self._prefixes)

    def forward(self, x: torch.Tensor, delta, step, cache: LayerCache):
        T = x.shape[0]
        h = self.env.workspace.get("block.normed", (T, self.hidden), self.env.dtype)
        self.mixer_norm.forward(x, h, delta=delta)
        delta = self.mixer.forward(h, step, cache)
        self.feed_forward_norm.forward(x, h, delta=delta)
        return self.feed_forward.forward(h, step)
