"""Device memory behind the cache manager's page ids and state slots.

One tensor per group, ``[runs, pages, *page_shape]``: a page id addresses the same page in
every run of the group.  What a page holds is the group's :class:`~allpaca_b200.parts.CacheNeed`;
for attention it is ``[2, kv_heads, page_size, head_dim]``: keys (index 0) then values (index 1),
the rows of one head contiguous.  The reference lays a page out as all K rows then all V rows
of one layer (crates/allpaca-core/src/kv_tier.rs:337-339, :577-580).
"""
from __future__ import annotations

from typing import Sequence

import torch


class GroupStorage:
    """Pages of one cache group for all the layer runs in it."""

    def __init__(self, num_runs: int, num_pages: int, page_shape: Sequence[int], dtype: torch.dtype,
                 device: torch.device):
        self.pages = torch.zeros((num_runs, num_pages, *[int(d) for d in page_shape]), dtype=dtype, device=device)

    def run_view(self, index: int) -> torch.Tensor:
        """``[pages, *page_shape]`` of one run."""
        return self.pages[index]

    def bytes(self) -> int:
        return self.pages.numel() * self.pages.element_size()


class StateStorage:
    """``[max_seqs, state_bytes]`` bytes per run that keeps fixed-size state."""

    def __init__(self, max_seqs: int, state_bytes: int, device: torch.device):
        self.rows = torch.zeros((max_seqs, max(int(state_bytes), 0)), dtype=torch.uint8, device=device)
