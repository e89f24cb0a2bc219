"""Cache pages, block tables and state slots: the Python face of the C++ cache manager.

The bookkeeping itself is C++ (``csrc/host/cache_manager.cpp``, built on first use with the
C++ compiler alone, so it runs where there is no GPU); this module maps request ids to
handles, turns status codes into exceptions and hands block tables back as lists.

Keys and values live in fixed-size pages.  Layers with the same need form a *group* with a
page pool of its own: a group either keeps every key of a request (``window`` None) or only a
trailing window of them, in which case pages the window has passed go back to the pool while
the request is still running.  Each request has, per group, a block table: logical page index
-> page id (``FREED`` where the page was given back).  Beside the pages there are slots for
per-request state of fixed size, one per running request, whatever the architecture keeps in
them.

Role in the reference: ``KvTierManager`` (crates/allpaca-core/src/kv_tier.rs:341-474,
:498-532), the per-request page lists released on drop (crates/allpaca-core/src/engine.rs:97,
:409-432), ``ensure_pages`` (crates/allpaca-core/src/model.rs:13452-13480) and the per-request
recurrent state (crates/allpaca-core/src/anchors.rs:16-56).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int64, c_void_p, c_char_p
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

FREED = -1
_OK, _MISUSE, _OUT_OF_PAGES = 0, 1, 2


class CacheError(RuntimeError):
    """Misuse of the cache manager (a bug in the caller)."""


class OutOfPages(RuntimeError):
    """A group's pool cannot supply the pages asked for; nothing was changed."""


_lib = None


def host_library() -> ctypes.CDLL:
    """The C++ host library, built on first use."""
    global _lib
    if _lib is None:
        from ..csrc import build
        lib = ctypes.CDLL(build.build_host())
        lib.apc_last_error.restype = c_char_p
        lib.apc_pool_create.restype = c_void_p
        lib.apc_pool_create.argtypes = [c_int]
        for name in ("apc_pool_destroy",):
            getattr(lib, name).argtypes = [c_void_p]
            getattr(lib, name).restype = None
        for name, args in {
            "apc_pool_alloc": [c_void_p], "apc_pool_free": [c_void_p, c_int], "apc_pool_num_free": [c_void_p],
            "apc_pool_held": [c_void_p, c_int],
            "apc_cache_begin": [c_void_p, c_int64, POINTER(c_int)], "apc_cache_free": [c_void_p, c_int64],
            "apc_cache_has": [c_void_p, c_int64], "apc_cache_num_running": [c_void_p],
            "apc_cache_can_begin": [c_void_p], "apc_cache_num_free_pages": [c_void_p, c_int],
            "apc_cache_state_slot": [c_void_p, c_int64],
            "apc_cache_pages_missing": [c_void_p, c_int64, c_int64, POINTER(c_int)],
            "apc_cache_can_append": [c_void_p, c_int64, c_int64, POINTER(c_int)],
            "apc_cache_append": [c_void_p, c_int64, c_int64, POINTER(c_int64)],
            "apc_cache_release_passed": [c_void_p, c_int64, POINTER(c_int)], "apc_cache_check": [c_void_p],
            "apc_cache_table": [c_void_p, c_int64, c_int, POINTER(c_int), c_int],
        }.items():
            getattr(lib, name).argtypes = args
            getattr(lib, name).restype = c_int
        lib.apc_cache_num_tokens.argtypes = [c_void_p, c_int64]
        lib.apc_cache_num_tokens.restype = c_int64
        lib.apc_cache_create.argtypes = [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), c_int]
        lib.apc_cache_create.restype = c_void_p
        lib.apc_cache_destroy.argtypes = [c_void_p]
        lib.apc_cache_destroy.restype = None
        lib.apc_prepare_step.argtypes = [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                         c_void_p, c_void_p]
        lib.apc_prepare_step.restype = c_int
        lib.aps_create.argtypes = [c_void_p, c_int, c_int64, c_int64, c_int64]
        lib.aps_create.restype = c_void_p
        lib.aps_destroy.argtypes = [c_void_p]
        lib.aps_destroy.restype = None
        for name, args in {
            "aps_add": [c_void_p, c_int64, c_int64, c_int64, POINTER(c_int), c_int],
            "aps_adopt_running": [c_void_p, c_int64, c_int64, c_int64, c_int64],
            "aps_has_unfinished": [c_void_p], "aps_schedule": [c_void_p, POINTER(c_int)],
            "aps_advance": [c_void_p, POINTER(c_int), c_int, POINTER(c_int)], "aps_abort": [c_void_p, c_int64],
            "aps_advance_counts": [c_void_p], "aps_resolve": [c_void_p, POINTER(c_int), c_int, POINTER(c_int)],
            "aps_unresolved_steps": [c_void_p],
            "aps_list": [c_void_p, c_int, POINTER(c_int64), c_int],
        }.items():
            getattr(lib, name).argtypes = args
            getattr(lib, name).restype = c_int
        lib.aps_planned.argtypes = [c_void_p, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64)]
        lib.aps_planned.restype = None
        lib.aps_finished.argtypes = [c_void_p, POINTER(c_int64), POINTER(c_int)]
        lib.aps_finished.restype = None
        # safetensors files (weights/safetensors_io.py is their Python face)
        lib.apst_open.argtypes = [c_char_p]
        lib.apst_open.restype = c_void_p
        lib.apst_close.argtypes = [c_void_p]
        lib.apst_close.restype = None
        for name in ("apst_num_tensors", "apst_num_metadata"):
            getattr(lib, name).argtypes = [c_void_p]
            getattr(lib, name).restype = c_int
        for name in ("apst_name", "apst_dtype", "apst_metadata_key", "apst_metadata_value"):
            getattr(lib, name).argtypes = [c_void_p, c_int]
            getattr(lib, name).restype = c_char_p
        lib.apst_ndim.argtypes = [c_void_p, c_int]
        lib.apst_ndim.restype = c_int
        lib.apst_shape.argtypes = [c_void_p, c_int, POINTER(c_int64), c_int]
        lib.apst_shape.restype = c_int
        for name in ("apst_begin", "apst_end"):
            getattr(lib, name).argtypes = [c_void_p, c_int]
            getattr(lib, name).restype = c_int64
        lib.apst_data.argtypes = [c_void_p]
        lib.apst_data.restype = c_void_p
        lib.apst_data_len.argtypes = [c_void_p]
        lib.apst_data_len.restype = c_int64
        _lib = lib
    return _lib


def _raise(status: int, what: str = "") -> None:
    msg = host_library().apc_last_error().decode() or what
    if what and what not in msg:
        msg = f"{what}: {msg}"
    if status == _OUT_OF_PAGES:
        raise OutOfPages(msg)
    raise CacheError(msg)


class PagePool:
    """Page ids ``0 .. n-1`` with a last-in-first-out free list, so a page that was just
    given back is the next one handed out."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self._lib = host_library()
        self._h = self._lib.apc_pool_create(self.num_pages)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.apc_pool_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.apc_pool_num_free(self._h)

    def alloc(self) -> int:
        p = self._lib.apc_pool_alloc(self._h)
        if p < 0:
            raise OutOfPages("the page pool is empty")
        return p

    def free(self, page: int) -> None:
        rc = self._lib.apc_pool_free(self._h, int(page))
        if rc != _OK:
            _raise(rc)

    def held(self) -> List[int]:
        return [p for p in range(self.num_pages) if self._lib.apc_pool_held(self._h, p)]


@dataclass(frozen=True)
class GroupLayout:
    """One cache group: its page size, pool size and window (None: keep everything)."""

    page_size: int
    num_pages: int
    window: Optional[int] = None


class CacheManager:
    """Pages, block tables and state slots of all running requests."""

    def __init__(self, groups: Sequence[GroupLayout], max_seqs: int):
        if max_seqs <= 0:
            raise CacheError("max_seqs must be positive")
        for g in groups:
            if g.page_size <= 0:
                raise CacheError("page_size must be positive")
            if g.num_pages <= 0:
                raise CacheError(f"a page pool needs at least one page, got {g.num_pages}")
            if g.window is not None and g.window <= 0:
                raise CacheError("a window must be positive")
        self.groups = list(groups)
        self.max_seqs = int(max_seqs)
        self._lib = host_library()
        n = len(self.groups)
        arr = c_int * max(n, 1)
        self._h = self._lib.apc_cache_create(
            n, arr(*[g.page_size for g in self.groups]), arr(*[g.num_pages for g in self.groups]),
            arr(*[(g.window or -1) for g in self.groups]), self.max_seqs)
        if not self._h:
            raise CacheError("the cache manager could not be created")
        self._handles: Dict[Hashable, int] = {}      # requests that hold cache -> their number
        self._numbers: Dict[Hashable, int] = {}      # every request that has been given a number
        self._pinned = set()                          # numbers a scheduler keeps across preemption
        self._next = 0
        self._ints = (c_int * max(n, 1))()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.apc_cache_destroy(self._h)
            self._h = None

    # ---- handles ----------------------------------------------------------
    def handle(self, req: Hashable) -> int:
        """The integer the C++ side knows a request by (-1: it holds no cache)."""
        return self._handles.get(req, -1)

    @property
    def native(self) -> int:
        """The C++ object, for other native code (the step builder)."""
        return self._h

    def number(self, req: Hashable) -> int:
        """The number native code knows the request by, given out on first asking.  It stays the
        same until the request's cache is freed (or, when pinned, until it is unpinned)."""
        n = self._numbers.get(req)
        if n is None:
            n = self._numbers[req] = self._next
            self._next += 1
        return n

    def pin(self, req: Hashable) -> int:
        """Keep the request's number across :meth:`free` (a scheduler that may preempt and
        recompute it); returns the number."""
        n = self.number(req)
        self._pinned.add(req)
        return n

    def unpin(self, req: Hashable) -> None:
        self._pinned.discard(req)
        if req not in self._handles:
            self._numbers.pop(req, None)

    def _need(self, req: Hashable) -> int:
        try:
            return self._handles[req]
        except KeyError:
            raise CacheError(f"request {req!r} holds no cache") from None

    # ---- requests ---------------------------------------------------------
    def has(self, req: Hashable) -> bool:
        return req in self._handles

    def num_running(self) -> int:
        return len(self._handles)

    def can_begin(self) -> bool:
        return bool(self._lib.apc_cache_can_begin(self._h))

    def begin(self, req: Hashable) -> int:
        """Register a request and give it a state slot.  Returns the slot."""
        if req in self._handles:
            raise CacheError(f"request {req!r} already holds a cache")
        known = req in self._numbers
        h = self.number(req)
        slot = c_int(-1)
        rc = self._lib.apc_cache_begin(self._h, h, ctypes.byref(slot))
        if rc != _OK:
            if not known:
                self._numbers.pop(req, None)
            _raise(rc)
        self._handles[req] = h
        return slot.value

    def adopt(self, req: Hashable) -> int:
        """Reserve the handle a new request will get from native code that begins it
        (the step builder); returns it."""
        h = self.number(req)
        self._handles[req] = h
        return h

    def forget(self, req: Hashable) -> None:
        """Drop a handle reserved with :meth:`adopt` whose request never began, or one whose
        cache native code has freed itself (a preemption by the scheduler)."""
        self._handles.pop(req, None)
        if req not in self._pinned:
            self._numbers.pop(req, None)

    def free(self, req: Hashable) -> None:
        """Give back everything the request holds."""
        h = self._handles.pop(req, None)
        if h is None:
            raise CacheError(f"request {req!r} holds no cache (freed twice?)")
        if req not in self._pinned:
            self._numbers.pop(req, None)
        rc = self._lib.apc_cache_free(self._h, h)
        if rc != _OK:
            _raise(rc, f"request {req!r}")

    # ---- pages ------------------------------------------------------------
    def num_tokens(self, req: Hashable) -> int:
        return int(self._lib.apc_cache_num_tokens(self._h, self._need(req)))

    def state_slot(self, req: Hashable) -> int:
        return int(self._lib.apc_cache_state_slot(self._h, self._need(req)))

    def pages_missing(self, req: Optional[Hashable], num_new: int, have_tokens: int = 0) -> List[int]:
        """Pages each group still has to allocate so that ``num_new`` more tokens fit.
        ``req`` None asks for a request that has not begun."""
        h = -1 if req is None else self._need(req)
        rc = self._lib.apc_cache_pages_missing(self._h, h, int(num_new) + int(have_tokens), self._ints)
        if rc != _OK:
            _raise(rc)
        return [self._ints[g] for g in range(len(self.groups))]

    def can_append(self, req: Optional[Hashable], num_new: int, reserve: Optional[Sequence[int]] = None) -> bool:
        """Whether :meth:`append` would succeed.  ``reserve[g]`` pages of each pool are treated
        as already spoken for (by other requests of the same step)."""
        h = -1 if req is None else self._need(req)
        res = None
        if reserve is not None:
            res = (c_int * max(len(self.groups), 1))(*[int(r) for r in reserve])
        return bool(self._lib.apc_cache_can_append(self._h, h, int(num_new), res))

    def append(self, req: Hashable, num_new: int) -> int:
        """Make room for ``num_new`` more tokens and count them as held.  Returns the position
        of the first new token.  On :class:`OutOfPages` nothing has changed."""
        first = c_int64(0)
        rc = self._lib.apc_cache_append(self._h, self._need(req), int(num_new), ctypes.byref(first))
        if rc != _OK:
            _raise(rc, f"request {req!r}")
        return int(first.value)

    def release_passed(self, req: Hashable) -> int:
        """Give back pages of windowed groups that no later token of the request can see.
        Call after the step that computed the held tokens.  Returns pages freed."""
        freed = c_int(0)
        rc = self._lib.apc_cache_release_passed(self._h, self._need(req), ctypes.byref(freed))
        if rc != _OK:
            _raise(rc)
        return freed.value

    def has_windows(self) -> bool:
        return any(g.window is not None for g in self.groups)

    def block_table(self, req: Hashable, group: int) -> List[int]:
        h = self._need(req)
        n = self._lib.apc_cache_table(self._h, h, int(group), None, 0)
        if n < 0:
            raise CacheError(f"request {req!r} has no group {group}")
        buf = (c_int * max(n, 1))()
        self._lib.apc_cache_table(self._h, h, int(group), buf, n)
        return list(buf[:n])

    def slot(self, req: Hashable, group: int, position: int) -> int:
        """``page * page_size + offset`` of a held position; its page must be live."""
        P = self.groups[group].page_size
        table = self.block_table(req, group)
        j = position // P
        if j >= len(table) or table[j] == FREED:
            raise CacheError(f"position {position} of request {req!r} has no live page in group {group}")
        return table[j] * P + position % P

    def slots(self, req: Hashable, group: int, first: int, count: int) -> List[int]:
        P = self.groups[group].page_size
        table = self.block_table(req, group)
        out = []
        for pos in range(first, first + count):
            page = table[pos // P]
            if page == FREED:
                raise CacheError(f"position {pos} of request {req!r} lies in a page already given back")
            out.append(page * P + pos % P)
        return out

    # ---- inspection -------------------------------------------------------
    def num_free_pages(self, group: int = 0) -> int:
        return int(self._lib.apc_cache_num_free_pages(self._h, int(group)))

    def check(self) -> None:
        """Every page is either free or held by exactly one request."""
        rc = self._lib.apc_cache_check(self._h)
        if rc != _OK:
            _raise(rc)
        if self._lib.apc_cache_num_running(self._h) != len(self._handles):
            raise CacheError("the request table and the native cache manager disagree")
