"""Reader and writer for the safetensors container.

Format (as the reference parses it, crates/allpaca-safetensors/src/parser.rs:93-159
and :181-188): an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` with an optional
``__metadata__`` entry, then the tensor bytes; offsets count from the end of
the header.  Sharded checkpoints carry ``model.safetensors.index.json`` with a
``weight_map`` from tensor name to file (crates/allpaca-safetensors/src/catalog.rs:51-98).

Files are opened, checked and memory-mapped by the C++ host library
(``csrc/host/safetensors.cpp``); tensors are handed out as torch tensors over the
mapping in their stored dtype, nothing is converted here.  The writer (used by the
random-weights mode) is Python.
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
from typing import Dict, List, Mapping, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A safetensors file that cannot be read as such."""


class SafetensorsFile:
    """One memory-mapped safetensors file.  Opening, the header (length, UTF-8, JSON, every
    entry's type, shape and byte range) and the mapping are the C++ host library's
    (``csrc/host/safetensors.cpp``); this class hands the mapped bytes out as torch tensors."""

    def __init__(self, path: str):
        from ..cache.manager import host_library
        self.path = path
        self._lib = host_library()
        self._h = self._lib.apst_open(os.fsencode(path))
        if not self._h:
            raise SafetensorsError(self._lib.apc_last_error().decode("utf-8", "replace"))
        lib, h = self._lib, self._h
        self.metadata = {lib.apst_metadata_key(h, i).decode(): lib.apst_metadata_value(h, i).decode()
                         for i in range(lib.apst_num_metadata(h))}
        self._data = lib.apst_data(h) or 0
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for i in range(lib.apst_num_tensors(h)):
            nd = lib.apst_ndim(h, i)
            dims = (ctypes.c_int64 * max(nd, 1))()
            lib.apst_shape(h, i, dims, max(nd, 1))
            self.entries[lib.apst_name(h, i).decode()] = (
                _DTYPES[lib.apst_dtype(h, i).decode()], tuple(int(d) for d in dims[:nd]),
                int(lib.apst_begin(h, i)), int(lib.apst_end(h, i)))

    def __del__(self):
        # tensors handed out keep this object alive (see ``tensor``), so nothing reads the
        # mapping any more when it goes
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.apst_close(h)

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """The stored tensor as a read-only view of the mapping (copy before writing)."""
        dtype, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dtype)
        buf = (ctypes.c_char * (e - b)).from_address(self._data + b)
        buf._file = self                      # the view holds the buffer, the buffer holds the mapping
        t = torch.frombuffer(buf, dtype=dtype)
        return t.view(shape)


class Checkpoint:
    """All tensors of a model folder: one file, or shards named by an index."""

    def __init__(self, path: str):
        self.files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        for f in discover_weight_files(path):
            sf = SafetensorsFile(f)
            self.files.append(sf)
            for n in sf.names():
                if n in self._where:
                    raise SafetensorsError(
                        f"tensor {n!r} appears in both {self._where[n].path} and {f}")
                self._where[n] = sf

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str):
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)


def discover_weight_files(path: str) -> List[str]:
    """Index file, then ``model.safetensors``, then a single ``*.safetensors``
    (crates/allpaca-safetensors/src/catalog.rs:145-194)."""
    if os.path.isfile(path):
        return [path]
    if not os.path.isdir(path):
        raise SafetensorsError(f"no model folder or file at {path}")
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map")
        if not isinstance(wm, dict) or not wm:
            raise SafetensorsError(f"{index} has no weight_map")
        return [os.path.join(path, n) for n in sorted(set(wm.values()))]
    single = os.path.join(path, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    found = sorted(n for n in os.listdir(path) if n.endswith(".safetensors"))
    if len(found) == 1:
        return [os.path.join(path, found[0])]
    if not found:
        raise SafetensorsError(f"no .safetensors file in {path}")
    raise SafetensorsError(
        f"{path} holds several .safetensors files and no index: {', '.join(found)}")


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors (moved to the CPU, made contiguous) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    items = []
    for name in sorted(tensors):
        t = tensors[name].detach().to("cpu").contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype} that safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        items.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
