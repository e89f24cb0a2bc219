"""Bookkeeping of cache pages, block tables and state slots (host side, no tensors).

Keys and values live in fixed-size pages.  Layers with the same need form a *group*
with a page pool of its own: a group either keeps every key of a request (``window``
None) or only a trailing window of them, in which case pages the window has passed
go back to the pool while the request is still running.  Each request has, per
group, a block table: logical page index -> page id (``FREED`` where the page was
given back).  Beside the pages there are slots for per-request state of fixed size,
one per running request, whatever the architecture keeps in them.

Role in the reference: ``KvTierManager`` page allocation and release
(crates/allpaca-core/src/kv_tier.rs:341-474, :498-532), the per-request page lists of
``ActiveRequest`` (crates/allpaca-core/src/engine.rs:97) released on drop
(engine.rs:409-432), growth by ``ensure_pages`` (crates/allpaca-core/src/model.rs:13452-13480)
and the per-request recurrent state (crates/allpaca-core/src/anchors.rs:16-56).  The
reference allocates a page per layer and evicts to slower tiers when VRAM is full;
here one page id addresses the same page in every layer of its group, there is one
tier, and running out of pages is reported to the scheduler.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

FREED = -1


class CacheError(RuntimeError):
    """Misuse of the cache manager (a bug in the caller)."""


class OutOfPages(RuntimeError):
    """A group's pool cannot supply the pages asked for; nothing was changed."""


class PagePool:
    """Page ids ``0 .. n-1`` with a last-in-first-out free list, so a page that was just
    given back is the next one handed out."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("the page pool is empty")
        p = self._free.pop()
        if self._held[p]:
            raise CacheError(f"page {p} was on the free list while held")
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} is outside the pool of {self.num_pages}")
        if not self._held[page]:
            raise CacheError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)

    def held(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


@dataclass(frozen=True)
class GroupLayout:
    """One cache group: its page size, pool size and window (None: keep everything)."""

    page_size: int
    num_pages: int
    window: Optional[int] = None


@dataclass
class _Sequence:
    tables: List[List[int]]
    num_tokens: int = 0
    state_slot: int = -1


class CacheManager:
    """Pages, block tables and state slots of all running requests."""

    def __init__(self, groups: Sequence[GroupLayout], max_seqs: int):
        if max_seqs <= 0:
            raise CacheError("max_seqs must be positive")
        for g in groups:
            if g.page_size <= 0:
                raise CacheError("page_size must be positive")
            if g.window is not None and g.window <= 0:
                raise CacheError("a window must be positive")
        self.groups = list(groups)
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.max_seqs = int(max_seqs)
        self._free_slots: List[int] = list(range(self.max_seqs - 1, -1, -1))
        self._seqs: Dict[Hashable, _Sequence] = {}

    # ---- requests -------------------------------------------------------
    def has(self, req: Hashable) -> bool:
        return req in self._seqs

    def num_running(self) -> int:
        return len(self._seqs)

    def can_begin(self) -> bool:
        return bool(self._free_slots)

    def begin(self, req: Hashable) -> int:
        """Register a request and give it a state slot.  Returns the slot."""
        if req in self._seqs:
            raise CacheError(f"request {req!r} already holds a cache")
        if not self._free_slots:
            raise OutOfPages("every state slot is taken")
        slot = self._free_slots.pop()
        self._seqs[req] = _Sequence(tables=[[] for _ in self.groups], state_slot=slot)
        return slot

    def free(self, req: Hashable) -> None:
        """Give back everything the request holds."""
        seq = self._seqs.pop(req, None)
        if seq is None:
            raise CacheError(f"request {req!r} holds no cache (freed twice?)")
        for g, table in enumerate(seq.tables):
            for page in reversed(table):
                if page != FREED:
                    self.pools[g].free(page)
        self._free_slots.append(seq.state_slot)

    # ---- pages ----------------------------------------------------------
    def num_tokens(self, req: Hashable) -> int:
        return self._seq(req).num_tokens

    def state_slot(self, req: Hashable) -> int:
        return self._seq(req).state_slot

    def pages_missing(self, req: Optional[Hashable], num_new: int, have_tokens: int = 0) -> List[int]:
        """Pages each group still has to allocate so that ``num_new`` more tokens fit.
        ``req`` None asks for a request that has not begun (``have_tokens`` = 0)."""
        out = []
        for g, layout in enumerate(self.groups):
            if req is None:
                have_pages, total = 0, have_tokens + num_new
            else:
                seq = self._seq(req)
                have_pages, total = len(seq.tables[g]), seq.num_tokens + num_new
            need = -(-total // layout.page_size)
            out.append(max(0, need - have_pages))
        return out

    def can_append(self, req: Optional[Hashable], num_new: int, reserve: Optional[Sequence[int]] = None) -> bool:
        """Whether :meth:`append` would succeed.  ``reserve[g]`` pages of each pool are
        treated as already spoken for (by other requests of the same step)."""
        for g, miss in enumerate(self.pages_missing(req, num_new)):
            taken = reserve[g] if reserve is not None else 0
            if miss > self.pools[g].num_free - taken:
                return False
        return True

    def append(self, req: Hashable, num_new: int) -> int:
        """Make room for ``num_new`` more tokens and count them as held.  Returns the
        position of the first new token.  On :class:`OutOfPages` nothing has changed."""
        if num_new <= 0:
            raise CacheError("append needs at least one token")
        seq = self._seq(req)
        missing = self.pages_missing(req, num_new)
        for g, miss in enumerate(missing):
            if miss > self.pools[g].num_free:
                raise OutOfPages(
                    f"group {g} needs {miss} more pages for request {req!r}, "
                    f"{self.pools[g].num_free} are free")
        for g, miss in enumerate(missing):
            for _ in range(miss):
                seq.tables[g].append(self.pools[g].alloc())
        first = seq.num_tokens
        seq.num_tokens += num_new
        return first

    def release_passed(self, req: Hashable) -> int:
        """Give back pages of windowed groups that no later token of the request can
        see.  Call after the step that computed the held tokens.  Returns pages freed."""
        seq = self._seq(req)
        freed = 0
        for g, layout in enumerate(self.groups):
            if layout.window is None:
                continue
            # the next row sits at position num_tokens and sees keys > num_tokens - window
            first_visible = seq.num_tokens - layout.window + 1
            if first_visible <= 0:
                continue
            dead_pages = min(first_visible // layout.page_size, len(seq.tables[g]))
            table = seq.tables[g]
            for j in range(dead_pages):
                if table[j] != FREED:
                    self.pools[g].free(table[j])
                    table[j] = FREED
                    freed += 1
        return freed

    def block_table(self, req: Hashable, group: int) -> List[int]:
        return self._seq(req).tables[group]

    def slot(self, req: Hashable, group: int, position: int) -> int:
        """``page * page_size + offset`` of a held position; its page must be live."""
        layout = self.groups[group]
        table = self._seq(req).tables[group]
        j = position // layout.page_size
        if j >= len(table) or table[j] == FREED:
            raise CacheError(f"position {position} of request {req!r} has no live page in group {group}")
        return table[j] * layout.page_size + position % layout.page_size

    def slots(self, req: Hashable, group: int, first: int, count: int) -> List[int]:
        layout = self.groups[group]
        table = self._seq(req).tables[group]
        P = layout.page_size
        out = []
        for pos in range(first, first + count):
            page = table[pos // P]
            if page == FREED:
                raise CacheError(f"position {pos} of request {req!r} lies in a page already given back")
            out.append(page * P + pos % P)
        return out

    # ---- inspection -----------------------------------------------------
    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def check(self) -> None:
        """Every page is either free or held by exactly one request."""
        for g, pool in enumerate(self.pools):
            owners: Dict[int, Hashable] = {}
            for req, seq in self._seqs.items():
                for page in seq.tables[g]:
                    if page == FREED:
                        continue
                    if page in owners:
                        raise CacheError(f"page {page} of group {g} is held by {owners[page]!r} and {req!r}")
                    owners[page] = req
            held = set(pool.held())
            if held != set(owners):
                raise CacheError(f"group {g}: pool holds {sorted(held)}, requests hold {sorted(owners)}")
            if len(held) + pool.num_free != pool.num_pages:
                raise CacheError(f"group {g}: {len(held)} held + {pool.num_free} free != {pool.num_pages}")
        slots = [s.state_slot for s in self._seqs.values()]
        if len(set(slots)) != len(slots) or len(slots) + len(self._free_slots) != self.max_seqs:
            raise CacheError("state slots are lost or held twice")

    def _seq(self, req: Hashable) -> _Sequence:
        try:
            return self._seqs[req]
        except KeyError:
            raise CacheError(f"request {req!r} holds no cache") from None
