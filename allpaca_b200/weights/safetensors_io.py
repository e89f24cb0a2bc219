"""Reader and writer for the safetensors container.

Format (as the reference parses it, crates/allpaca-safetensors/src/parser.rs:93-159
and :181-188): an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` with an optional
``__metadata__`` entry, then the tensor bytes; offsets count from the end of
the header.  Sharded checkpoints carry ``model.safetensors.index.json`` with a
``weight_map`` from tensor name to file (crates/allpaca-safetensors/src/catalog.rs:51-98).

Tensors are memory-mapped and handed out as torch tensors in their stored
dtype; nothing is converted here.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Mapping, Optional, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024   # parser.rs:11

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A safetensors file that cannot be read as such."""


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a header length")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen == 0 or hlen > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: header length {hlen} is outside 1..{MAX_HEADER_BYTES}")
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header of {hlen} bytes overruns the file of {size} bytes")
        raw = self._fh.read(hlen)
        try:
            header = json.loads(raw.decode("utf-8"))
        except UnicodeDecodeError:
            raise SafetensorsError(f"{path}: header is not UTF-8") from None
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + hlen
        self._data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            dtype = _DTYPES[dt]
            n = 1
            for s in shape:
                n *= s
            need = n * torch.empty((), dtype=dtype).element_size()
            if not (0 <= b <= en <= self._data_len):
                raise SafetensorsError(
                    f"{path}: tensor {name!r} data [{b}, {en}) lies outside the {self._data_len} data bytes")
            if en - b != need:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} {dt} needs {need} bytes, has {en - b}")
            self.entries[name] = (dtype, shape, int(b), int(en))
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

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
        buf = memoryview(self._mm)[self._data_start + b:self._data_start + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # torch warns that the buffer is not writable
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
