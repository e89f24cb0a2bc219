"""A decoder built from a :class:`ModelSpec`: embedding, blocks in their order, final
norm on the wanted rows, head.

The model owns the parts and their weights; the engine owns the caches and hands each
run of the order a :class:`LayerCache`.  ``forward(step)`` runs exactly the rows of the
step and returns 32-bit logits for ``step.logit_rows``.

Role in the reference: ``forward_tokens_device_impl``
(crates/allpaca-core/src/model.rs:10836-11708): shared matrix products over all rows,
per-sequence rotation, cache write and attention, logits for chosen rows
(:11609-11636, :11665-11687).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import ops
from ..parts import (Block, BuildEnv, CacheNeed, Deferred, LayerCache, ModelSpec, Part, WeightSpec, build)
from ..parts.linear import Linear


@dataclass
class CacheGroupPlan:
    """Runs of the order that share a page pool, and what a page of theirs holds."""

    need: CacheNeed
    runs: List[int]


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.blocks: List[Block] = [build("block", b, env) for b in spec.layers]
        self.final_norm = build("norm", spec.final_norm, env)
        self.embedding: Optional[torch.Tensor] = None
        self.head = Linear(env, spec.vocab_size, spec.hidden_size)
        self.head_bias: Optional[torch.Tensor] = None
        self._validate_order()
        self.caches: List[LayerCache] = [LayerCache() for _ in spec.order]
        self._group_pages: List[Tuple[torch.Tensor, int]] = []

    def _validate_order(self) -> None:
        for r, run in enumerate(self.spec.order):
            if not (0 <= run.layer < len(self.blocks)):
                raise ValueError(f"order[{r}] names layer {run.layer}, there are {len(self.blocks)}")
            if run.cache_from is not None and not (0 <= run.cache_from < r):
                raise ValueError(f"order[{r}] reads the cache of entry {run.cache_from}, "
                                 f"which does not run before it")

    # ---- weights --------------------------------------------------------
    def weight_targets(self) -> Dict[str, Tuple[WeightSpec, Optional[Part], str]]:
        """Checkpoint tensor name -> (what it is, the part it goes to, its local name)."""
        s = self.spec
        out: Dict[str, Tuple[WeightSpec, Optional[Part], str]] = {
            s.embedding_name: (WeightSpec((s.vocab_size, s.hidden_size), "embedding"), None, "embedding"),
            s.head_name: (WeightSpec((s.vocab_size, s.hidden_size), "linear",
                                     optional=True), None, "head"),
        }
        if s.head_bias_name:
            out[s.head_bias_name] = (WeightSpec((s.vocab_size,), "bias"), None, "head_bias")
        for name, ws in self.final_norm.weights().items():
            out[s.final_norm_prefix + name] = (ws, self.final_norm, name)
        for block, prefix in zip(self.blocks, s.layer_prefixes):
            for sub_prefix, part in block.sub_parts().items():
                for name, ws in part.weights().items():
                    out[prefix + sub_prefix + name] = (ws, part, name)
        return out

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Distribute already validated device tensors (checkpoint names) to the parts."""
        per_part: Dict[int, Tuple[Part, Dict[str, torch.Tensor]]] = {}
        for full, (ws, part, local) in self.weight_targets().items():
            if full not in tensors:
                continue
            if part is None:
                continue
            per_part.setdefault(id(part), (part, {}))[1][local] = tensors[full]
        for part, got in per_part.values():
            part.load(got)
        for block in self.blocks:
            block.finalize()
        s = self.spec
        self.embedding = tensors[s.embedding_name].contiguous()
        if s.tie_word_embeddings or s.head_name not in tensors:
            # tied by flag, or by absence as the reference does (model.rs:8006-8009)
            self.head.load(self.embedding)
        else:
            self.head.load(tensors[s.head_name])
        self.head_bias = tensors[s.head_bias_name].contiguous() if s.head_bias_name else None

    # ---- caches ---------------------------------------------------------
    def cache_plan(self) -> List[CacheGroupPlan]:
        """Group the runs that write keys and values by what they keep."""
        groups: List[CacheGroupPlan] = []
        for r, run in enumerate(self.spec.order):
            if run.cache_from is not None:
                continue
            need = self.blocks[run.layer].mixer.cache_need()
            if need is None:
                continue
            for g in groups:
                if g.need == need:
                    g.runs.append(r)
                    break
            else:
                groups.append(CacheGroupPlan(need, [r]))
        return groups

    def host_control(self) -> bool:
        """Whether any part decides on the host, step by step, what it launches (such a model's
        steps are not recorded as CUDA graphs)."""
        every = [p for b in self.blocks for p in b.parts()] + list(self.final_norm.parts())
        return any(p.host_control for p in every)

    def state_bytes(self) -> List[int]:
        """Fixed-size state bytes per request, for each run of the order."""
        return [self.blocks[run.layer].mixer.state_bytes() for run in self.spec.order]

    def bind_caches(self, plan: List[CacheGroupPlan], storages, states) -> None:
        """``storages[g]`` backs group ``g`` of ``plan``; ``states[r]`` is the state rows of
        run ``r`` or None."""
        where: Dict[int, Tuple[int, int]] = {}
        # (all pages of a group, index of the page-size dimension), for the clearing of fresh pages
        self._group_pages = [(storages[g].pages, 2 + len(grp.need.outer)) for g, grp in enumerate(plan)]
        for g, grp in enumerate(plan):
            for i, r in enumerate(grp.runs):
                where[r] = (g, i)
        for r, run in enumerate(self.spec.order):
            src = run.cache_from if run.cache_from is not None else r
            cache = LayerCache(writes=run.cache_from is None,
                               state=states[r].rows if states[r] is not None else None)
            if src in where:
                g, i = where[src]
                cache.pages = storages[g].run_view(i)
                cache.group = g
            self.caches[r] = cache

    # ---- one step -------------------------------------------------------
    def forward(self, step) -> torch.Tensor:
        T = step.num_tokens
        ws = self.env.workspace
        s = self.spec
        step.shared.clear()
        # pages that get their first token in this step: nothing of their last owner stays readable
        for g, (pages, page_dim) in enumerate(self._group_pages):
            ops.clear_page_tails(pages, page_dim, step.positions, step.token_seq, step.block_tables[g],
                                 step.context_lens)
        x = ws.get("model.residual", (T, s.hidden_size), torch.float32)
        ops.embed_gather(step.token_ids, self.embedding, x,
                         s.embedding_scale if s.embedding_scale is not None else 1.0)
        delta = None
        for r, run in enumerate(s.order):
            delta = self.blocks[run.layer].forward(x, delta, step, self.caches[r])
        R = step.num_logit_rows
        logits = ws.get("model.logits", (R, s.vocab_size), torch.float32)
        if R == 0:
            return logits            # a portion nobody wants logits of: the cache is written, that is all
        h = ws.get("model.final_normed", (R, s.hidden_size), self.env.dtype)
        if isinstance(delta, Deferred):
            delta = None                 # the last block has added into the residual itself
        self.final_norm.forward(x, h, delta=delta, rows=step.logit_rows)
        out = self.head.forward(h, "model.logits", "float32")
        if self.head_bias is not None or s.logit_scale is not None or s.logit_softcap:
            ops.logit_transform(out, self.head_bias, s.logit_scale if s.logit_scale is not None else 1.0,
                                s.logit_softcap or 0.0)
        return out
