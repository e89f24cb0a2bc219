"""Grouped-query causal attention over a paged cache.

Steps, as the reference computes them (crates/allpaca-core/src/model.rs:8528-8667):
``q = Wq h``, ``k = Wk h``, ``v = Wv h`` without bias (:8528-8560); Q and K (not V) of every
head are rotated at the token's absolute position (:8573-8604); K and V go into the
page ``pos / P`` at slot ``pos % P`` (:8606-8614); query head ``h`` reads KV head
``h / (heads/kv_heads)``, scores are ``(q.k) / sqrt(head_dim)`` over the keys at or before the
row's position (crates/allpaca-cpu/src/kernels.rs:318-336), soft-maxed and applied to the
values (:338-352); then ``Wo`` (model.rs:8667).  The three projections are one matrix
product here: their weights are stacked ``[Wq; Wk; Wv]`` at load.

A ``window`` keeps only the last ``window`` keys visible, and lets the cache manager take
back pages the window has passed.  ``shares_kv`` makes the layer read keys and values that
another run of the order wrote: it then has no K/V weights.
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import BuildEnv, CacheNeed, KVNeed, LayerCache, Mixer, PartError, WeightSpec, build, register
from .linear import Linear


@register("mixer", "gqa_attention")
class GroupedQueryAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``position`` (a :class:`PartSpec` of kind ``position`` or None), ``window`` (None or
    tokens), ``scale`` (None: ``1/sqrt(head_dim)``), ``shares_kv`` (False), ``qkv_bias`` and
    ``o_bias`` (False: the projections have no bias, as on the Llama path)."""

    #: rotation and cache store in the projection's epilogue for steps of few rows (a switch for
    #: measurements; the separate kernel gives the same results)
    FUSE_ROPE = True
    #: rows up to which that pays (8B shape, 1024 keys: 1 % of the step at 24 and 32 rows, a loss of
    #: 0.6 % at 64 and of 2 % at 128, where the epilogue's scattered stores hold the product up)
    FUSE_ROPE_MAX_ROWS = 32

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "num_heads", "num_kv_heads", "head_dim")
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} KV heads")
        if self.hd <= 0 or self.hd % 16 or self.hd > 256:
            raise PartError(f"head_dim {self.hd} is not one the attention kernels take (multiples of 16 up to 256)")
        self.window = p.get("window") or None
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.shares_kv = bool(p.get("shares_kv", False))
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.o_bias = bool(p.get("o_bias", False))
        pos = p.get("position")
        self.position = build("position", pos, env) if pos is not None else None
        self.q_size = self.nh * self.hd
        self.kv_size = 0 if self.shares_kv else self.nkv * self.hd
        self.qkv = Linear(env, self.q_size + 2 * self.kv_size, self.hidden)
        self.o = Linear(env, self.hidden, self.q_size)
        self._interleaved = False

    # ---- weights --------------------------------------------------------
    def weights(self) -> Dict[str, WeightSpec]:
        w = {"q_proj.weight": WeightSpec((self.q_size, self.hidden)),
             "o_proj.weight": WeightSpec((self.hidden, self.q_size))}
        if not self.shares_kv:
            w["k_proj.weight"] = WeightSpec((self.kv_size, self.hidden))
            w["v_proj.weight"] = WeightSpec((self.kv_size, self.hidden))
        if self.qkv_bias:
            w["q_proj.bias"] = WeightSpec((self.q_size,), "bias")
            if not self.shares_kv:
                w["k_proj.bias"] = WeightSpec((self.kv_size,), "bias")
                w["v_proj.bias"] = WeightSpec((self.kv_size,), "bias")
        if self.o_bias:
            w["o_proj.bias"] = WeightSpec((self.hidden,), "bias")
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        parts = [tensors["q_proj.weight"]]
        if not self.shares_kv:
            parts += [tensors["k_proj.weight"], tensors["v_proj.weight"]]
        # A rotation that pairs element j with j + hd/2 reaches, in a product's epilogue, only pairs
        # that lie side by side: where the products run on the tensor cores the rows of every Q
        # and K head are interleaved (row 2j: element j, row 2j+1: element j + hd/2), and the
        # kernels that rotate put the results back in their places.
        self._interleaved = False
        if (self.env.dtype == torch.bfloat16 and not self.shares_kv and not self.qkv_bias
                and getattr(self.position, "pairing", None) == 0
                and all(t.dtype == torch.bfloat16 for t in parts) and self.hidden % 8 == 0
                and ops.tensor_core_gemm_available()):
            half = self.hd // 2
            order = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
            for i in (0, 1):
                t = parts[i]
                heads = t.shape[0] // self.hd
                parts[i] = t.view(heads, self.hd, -1)[:, order.to(t.device), :].reshape(t.shape)
            self._interleaved = True
        names = ["q_proj"] + ([] if self.shares_kv else ["k_proj", "v_proj"])
        bias = torch.cat([tensors[n + ".bias"] for n in names], dim=0) if self.qkv_bias else None
        self.qkv.load(torch.cat(parts, dim=0) if len(parts) > 1 else parts[0], bias)
        self.o.load(tensors["o_proj.weight"], tensors["o_proj.bias"] if self.o_bias else None)

    # ---- cache ----------------------------------------------------------
    def cache_need(self) -> Optional[CacheNeed]:
        return KVNeed(self.nkv, self.hd, self.window)

    def parts(self):
        yield self
        if self.position is not None:
            yield from self.position.parts()

    # ---- the norm before, and the residual addition after, inside the products -----------
    def can_fold_input_norm(self) -> bool:
        """Whether the products can take the norm before this mixer as a scale of their result and
        add into the residual themselves."""
        return self.qkv.fusable() and self.o.fusable()

    def fold_input_norm(self, weight: torch.Tensor) -> None:
        """Multiply the weight of the norm before this mixer into the first product."""
        self.qkv.fold_input_scale(weight)

    def fused_rows_ok(self, T: int) -> bool:
        return T <= Linear.FUSED_MAX_ROWS and self.o.residual_rows_ok(T)

    def forward_fused(self, h: torch.Tensor, scale, x: torch.Tensor, step, cache: LayerCache):
        """Like :meth:`forward`, for few rows: ``h`` is the residual's bfloat16 copy with ``scale``
        (an ``ops.RowScale``) standing for the norm, or normed rows with ``scale`` None; the
        output projection adds into ``x`` itself.  Returns a :class:`Deferred`."""
        attn = self._attend(h, step, cache, scale)
        return self.o.forward_residual(attn, x, "attn")

    # ---- one step -------------------------------------------------------
    def forward(self, h: torch.Tensor, step, cache: LayerCache) -> torch.Tensor:
        return self.o.forward(self._attend(h, step, cache, None), "attn.o", "delta")

    def _attend(self, h: torch.Tensor, step, cache: LayerCache, scale) -> torch.Tensor:
        T = h.shape[0]
        ws = self.env.workspace
        q = ws.get("attn.q", (T, self.q_size), self.env.dtype)
        table = self.position.rotation_for(step) if self.position is not None else None
        writes = cache.writes and not self.shares_kv
        if (self.FUSE_ROPE and T <= self.FUSE_ROPE_MAX_ROWS and not self.shares_kv and self.qkv.fusable()
                and (self.position is None or table is not None) and (table is None or table[1] == 1 or self._interleaved)):
            # few rows: rotation and the store of keys and values in the projection's epilogue
            cos_sin, pairing = table if table is not None else (None, 1)
            ops.gemm_tc_rope(h, self.qkv.weight, q, cache.pages if writes else None, step.positions, step.token_seq,
                             step.block_tables[cache.group] if writes else None, cos_sin, pairing, self.nh,
                             self.nkv, self.hd, ops.gemm_tc_splits(T, self.qkv.out_features, self.hidden), scale)
            return self._attention(q, T, step, cache, ws)
        qkv = self.qkv.forward(h, "attn.qkv", "either", scale=scale)
        if self.position is not None and table is None:
            # an encoding that is not a plain rotation: let it act on views, then store
            qkv = self._materialise(qkv, T)
            qv = qkv[:, :self.q_size].unflatten(1, (self.nh, self.hd))
            kv = qkv[:, self.q_size:self.q_size + self.kv_size].unflatten(1, (-1, self.hd)) \
                if self.kv_size else None
            self.position.apply(qv, kv, step.positions)
        cos_sin, pairing = table if table is not None else (None, 0)
        if self._interleaved:
            pairing = 2                  # pairs side by side in the projection's output, halves in the result
        ops.rope_kv_store(
            qkv, q, cache.pages if writes else None, step.positions, step.token_seq,
            step.block_tables[cache.group] if writes else None, cos_sin, pairing,
            self.nh, self.nkv if not self.shares_kv else 0, self.hd)
        return self._attention(q, T, step, cache, ws)

    def _attention(self, q, T, step, cache, ws):
        attn = ws.get("attn.out", (T, self.q_size), self.env.dtype)
        ops.attention(q, attn, cache.pages, step.block_tables[cache.group], step.token_seq,
                      step.positions, self.nh, self.nkv, self.hd, self.scale,
                      self.window or 0, seq_start=step.seq_start, query_lens=step.host_query_lens,
                      max_context=step.max_decode_context_len or step.max_context_len, scratch=ws.get,
                      mean_context=step.mean_context_len)
        return attn

    def _materialise(self, qkv: torch.Tensor, T: int) -> torch.Tensor:
        """Partial sums -> one tensor in the activation type (rare path)."""
        if qkv.dim() == 2:
            return qkv
        return qkv.sum(dim=0).to(self.env.dtype)
