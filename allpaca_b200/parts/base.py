"""Interfaces and registries of the parts a decoder is assembled from.

A model is described by data (:class:`ModelSpec`): which mixer, feed-forward, norms
and block arrangement each layer has, with every size and constant as a parameter,
and the order in which layers run.  The classes behind the names are looked up in
the registries below; a part never learns which model it sits in.

Kinds of part and what each must provide
----------------------------------------
``mixer``         :class:`Mixer`        mixes information between the rows of a sequence
``feed_forward``  :class:`FeedForward`  acts on every row alone
``norm``          :class:`Norm`         adds the pending residual delta and normalises
``position``      :class:`PositionEncoding`  injects positions into queries and keys
``block``         :class:`Block`        arranges the parts above around the residual stream

All parts share :class:`Part`: ``weights()`` names the tensors they need (local
names, shapes, roles) and ``load()`` receives them.  A part is registered with
``@register(kind, name)`` and built with ``build(kind, spec, env)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

KINDS = ("mixer", "feed_forward", "norm", "position", "block")
_REGISTRY: Dict[str, Dict[str, type]] = {k: {} for k in KINDS}


class PartError(ValueError):
    pass


def register(kind: str, name: str) -> Callable[[type], type]:
    """Class decorator: make ``name`` buildable as a part of ``kind``."""
    if kind not in _REGISTRY:
        raise PartError(f"unknown kind of part {kind!r} (known: {', '.join(KINDS)})")

    def deco(cls: type) -> type:
        _REGISTRY[kind][name] = cls
        return cls
    return deco


def registered(kind: str) -> List[str]:
    return sorted(_REGISTRY[kind])


@dataclass(frozen=True)
class PartSpec:
    """The name of a registered part and its parameters."""

    name: str
    params: Mapping[str, Any] = field(default_factory=dict)


def build(kind: str, spec: PartSpec, env: "BuildEnv") -> "Part":
    try:
        cls = _REGISTRY[kind][spec.name]
    except KeyError:
        raise PartError(f"no {kind} named {spec.name!r} is registered "
                        f"(known: {', '.join(registered(kind)) or 'none'})") from None
    return cls(dict(spec.params), env)


@dataclass
class BuildEnv:
    """What a part needs to know about the engine it is built into."""

    dtype: torch.dtype                 # storage and activation type: bfloat16 or float32
    device: torch.device
    workspace: "Workspace"
    page_size: int = 16                # tokens per cache page
    max_seqs: int = 1                  # state slots available to mixers with fixed-size state


class Workspace:
    """Named scratch buffers that live as long as the engine and grow on demand.

    A buffer is asked for by name and shape on every step; the same memory comes
    back while the request fits, so steady-state steps allocate nothing.
    """

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}     # (name, shape, dtype) -> the view last handed out
        self.generation = 0          # grows whenever a buffer is replaced (its address changes)

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        vkey = (name, tuple(shape), dtype)
        view = self._views.get(vkey)
        if view is not None:
            return view                  # the same shape as before: the same view of the same memory
        n = 1
        for s in shape:
            n *= int(s)
        key = f"{name}:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            grow = max(n, 1)
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
            # views of the buffer this one replaces are stale
            self._views = {k: v for k, v in self._views.items() if not (k[0] == name and k[2] == dtype)}
        view = buf[:n].view(*shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[vkey] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part needs: its shape and what it is (decides type and random init)."""

    shape: Tuple[int, ...]
    role: str = "linear"      # "linear" | "embedding" | "norm" | "bias" | "table"
    optional: bool = False


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token, in pages.

    One page of one run of the order is a tensor ``[*outer, page_size, *inner]`` of ``dtype``
    (None: the engine's activation type): ``inner`` is what one token stores contiguously,
    ``outer`` counts separate planes of such rows inside a page (keys and values of several
    heads: ``(2, kv_heads)`` with ``inner = (head_dim,)``; one latent vector per token:
    ``()`` with ``inner = (width,)``).  ``window`` (None: every earlier token stays readable)
    lets the cache manager take back the pages a trailing window has passed.  Runs whose
    needs are equal share a page pool and a block table."""

    outer: Tuple[int, ...] = ()
    inner: Tuple[int, ...] = ()
    dtype: Optional[torch.dtype] = None
    window: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (*self.outer, int(page_size), *self.inner)

    def page_bytes(self, page_size: int, engine_dtype: torch.dtype) -> int:
        n = int(page_size)
        for d in (*self.outer, *self.inner):
            n *= int(d)
        return n * torch.empty((), dtype=self.dtype or engine_dtype).element_size()


def KVNeed(num_kv_heads: int, head_dim: int, window: Optional[int] = None) -> CacheNeed:
    """Keys and values of ``num_kv_heads`` heads per token: pages ``[2, kv_heads, page, head_dim]``."""
    return CacheNeed(outer=(2, int(num_kv_heads)), inner=(int(head_dim),), window=window)


@dataclass
class LayerCache:
    """What one run of a layer sees of the caches.

    ``pages``: pages of this run ``[num_pages, *outer, page_size, *inner]`` (see
    :class:`CacheNeed`) or None;
    ``group``: index into the step's per-group block tables;
    ``writes``: False when the run reads the pages another run wrote;
    ``state``: ``[max_seqs, state_bytes]`` uint8 rows of fixed-size state, or None.
    """

    pages: Optional[torch.Tensor] = None
    group: int = -1
    writes: bool = True
    state: Optional[torch.Tensor] = None


@dataclass
class Deferred:
    """What a block that fuses its norms into the neighbouring products hands on instead of a
    32-bit delta: the residual is already updated; ``xb`` is its bfloat16 copy and ``ss [T, parts]``
    the partial sums of squares of its rows, from which the next product scales its result."""

    xb: torch.Tensor
    ss: torch.Tensor
    parts: int


class Part:
    """Common face of every part."""

    #: True when ``forward`` reads the step's host-side lists (``step.host_*``) or otherwise
    #: decides on the host what to launch for a given step.  Steps of a model with such a
    #: part are never recorded as CUDA graphs: a replay would repeat the decisions of the
    #: recorded step.  A part that reads only the step's device tensors (``state_slots``,
    #: ``seq_start``, ``positions`` ...; a sequence's first portion is the one whose first row
    #: has position 0) leaves it False.
    host_control: bool = False

    def __init__(self, params: Dict[str, Any], env: BuildEnv):
        self.params = params
        self.env = env

    def parts(self):
        """This part and the parts built inside it."""
        yield self

    def weights(self) -> Dict[str, WeightSpec]:
        """Local tensor names -> what they are."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors named by :meth:`weights`, already on the device."""

    def require(self, *names: str) -> None:
        missing = [n for n in names if n not in self.params]
        if missing:
            raise PartError(f"{type(self).__name__} lacks parameters {missing}")


class Norm(Part):
    """``forward(x, out, delta, rows)``: add ``delta`` (32-bit partial sums or None) into the
    32-bit residual ``x`` and write the normalised rows to ``out``.  With ``rows`` only those
    rows are produced and ``x`` is left untouched."""

    def forward(self, x, out, delta=None, rows=None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """Injects positions into queries and keys.

    ``rotation_for(step)`` returns ``(cos_sin [T, head_dim/2, 2] float32, pairing)`` when the
    encoding is a rotation the fused rotate-and-store kernel can apply, else None; then
    ``apply`` is called on ``q [T, heads, hd]`` and ``k [T, kv_heads, hd]`` views in place
    before keys are stored.
    """

    def rotation_for(self, step):
        return None

    def apply(self, q, k, positions) -> None:
        raise NotImplementedError


class Mixer(Part):
    """``forward(h, step, cache) -> delta``: ``h [T, hidden]`` normalised rows in the activation
    type; returns 32-bit ``[S, T, hidden]`` partial sums to be added to the residual."""

    def cache_need(self) -> Optional[CacheNeed]:
        """What the mixer keeps per token in pages (None: nothing)."""
        return None

    def state_bytes(self) -> int:
        """Bytes of fixed-size state per request (0: none)."""
        return 0

    def forward(self, h, step, cache: LayerCache):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(h, step) -> delta`` with the same shapes as a mixer."""

    def forward(self, h, step):
        raise NotImplementedError


class Block(Part):
    """Arrangement of mixer, feed-forward and norms around the residual stream.

    ``forward(x, delta, step, cache) -> delta``: ``x`` is the 32-bit residual ``[T, hidden]``,
    ``delta`` the pending addition of the previous block (None for the first); the block adds
    it (inside its first norm) and returns its own last pending addition.
    """

    mixer: Mixer

    def sub_parts(self) -> Dict[str, Part]:
        """Weight-name prefix -> part, for loading."""
        raise NotImplementedError

    def parts(self):
        yield self
        for part in self.sub_parts().values():
            yield from part.parts()

    def forward(self, x, delta, step, cache: LayerCache):
        raise NotImplementedError

    def finalize(self) -> None:
        """Called once every part of the block has its weights: the place to precompute what
        spans parts (a norm's weight multiplied into the product that follows it)."""


# ---------------------------------------------------------------------------
# whole-model description
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run ``layer``; ``cache_from`` names an earlier entry
    of the order whose keys and values this run reads instead of writing its own."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A decoder as data: parts per layer, the order they run in, and the ends."""

    hidden_size: int
    vocab_size: int
    layers: Tuple[PartSpec, ...]                 # block specs, one per distinct layer
    layer_prefixes: Tuple[str, ...]              # checkpoint prefix of each layer's tensors
    order: Tuple[LayerRun, ...]
    final_norm: PartSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 2048
    # Ends of the stack that some decoders alter; all default to "as it is".
    embedding_scale: Optional[float] = None      # the gathered embedding row is multiplied by it
    head_bias_name: Optional[str] = None         # a [vocab] tensor added to the logits
    logit_scale: Optional[float] = None          # logits are multiplied by it ...
    logit_softcap: Optional[float] = None        # ... and then become cap * tanh(logit / cap)
