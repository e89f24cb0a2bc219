"""Builds the CUDA kernel libraries of this package with nvcc, for sm_100a only.

Three kinds of shared library are produced, each from the sources in this folder:

* ``host``: the C++ host code (cache manager, step builder), built with the C++ compiler
  alone, so it also builds and is tested where there is no GPU.
* ``core``: every kernel that does not depend on a model size known only at run
  time (row-wise kernels, matrix products, sampling).
* ``attn<HD>``: the attention kernels specialised for one head size, built on
  first use for the head size of the model being loaded.

Objects and libraries live in ``allpaca_b200/_build`` (or, when the package folder
cannot be written, in a per-user folder under the system's temporary directory).
A library is rebuilt when the text of any of its sources or the flags change.
While nvcc runs, a progress line goes to standard error every few seconds.

Role in the reference: the nvcc discovery and static-library build of
crates/allpaca-cuda/build.rs:54-86 and :304-371.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Sequence

CSRC = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(CSRC)

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

CORE_SOURCES = ["errors.cu", "elementwise.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "gemm_pair.cu",
                "sampling.cu", "sampling_cluster.cu"]
ATTN_SOURCES = ["errors.cu", "attention.cu", "attention_tc.cu", "attention_tcgen05.cu",
                "attention_tcgen05_wide.cu"]
HEADERS = ["common.cuh", "tcgen05.cuh", "attention_noalloc.h"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("ALLPACA_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $ALLPACA_NVCC, $CUDA_HOME/bin, "
                     "/usr/local/cuda/bin and PATH); the CUDA kernels cannot be built")


def build_dir() -> str:
    override = os.environ.get("ALLPACA_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    d = os.path.join(PACKAGE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"allpaca_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _existing(names: Sequence[str]) -> List[str]:
    return [n for n in names if os.path.isfile(os.path.join(CSRC, n))]


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for n in list(sources) + _existing(HEADERS):
        with open(os.path.join(CSRC, n), "rb") as f:
            h.update(n.encode())
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


class _Progress:
    """Prints a line now and then while a build runs."""

    def __init__(self, what: str):
        self.what = what
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t0 = time.time()

    def _run(self):
        while not self._stop.wait(5.0):
            print(f"[allpaca_b200] still compiling {self.what} ({time.time() - self._t0:.0f} s)",
                  file=sys.stderr, flush=True)

    def __enter__(self):
        print(f"[allpaca_b200] compiling {self.what} ", file=sys.stderr, flush=True)
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._t.join()
        if exc[0] is None:
            print(f"[allpaca_b200] compiled {self.what} in {time.time() - self._t0:.0f} s",
                  file=sys.stderr, flush=True)


def _run(cmd: List[str]) -> str:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError("command failed: " + " ".join(cmd) + "\n" + p.stdout)
    return p.stdout


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = (),
                  verbose: bool = False) -> str:
    """Compile `sources` into ``lib<name>.so`` and return its path (cached by content)."""
    sources = _existing(sources)
    flags = ARCH_FLAGS + COMMON_FLAGS + [f"-D{d}" for d in defines]
    if verbose:
        flags = flags + ["-Xptxas", "-v"]
    tag = _digest(sources, flags)
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"lib{name}.{tag}.so")
    if os.path.isfile(lib):
        return lib
    nvcc = find_nvcc()
    obj_dir = os.path.join(out_dir, f"obj_{name}_{tag}_{os.getpid()}")
    os.makedirs(obj_dir, exist_ok=True)
    log = []
    with _Progress(f"{name} ({', '.join(sources)})"):
        def one(src: str) -> str:
            obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
            log.append(_run([nvcc] + flags + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]))
            return obj
        with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 2)) as ex:
            objs = list(ex.map(one, sources))
        tmp = lib + f".tmp{os.getpid()}"
        _run([nvcc, "-shared", "-o", tmp] + objs + ["-lcudart"])
        os.replace(tmp, lib)           # atomic: concurrent builders cannot see half a file
    shutil.rmtree(obj_dir, ignore_errors=True)
    if verbose:
        print("".join(log), file=sys.stderr)
    # keep only the newest build of this library
    for f in os.listdir(out_dir):
        if f.startswith(f"lib{name}.") and f.endswith(".so") and f != os.path.basename(lib):
            try:
                os.remove(os.path.join(out_dir, f))
            except OSError:
                pass
    return lib


HOST_SOURCES = ["host/cache_manager.cpp", "host/step_builder.cpp", "host/scheduler.cpp", "host/safetensors.cpp",
                "host/c_api.cpp"]
HOST_HEADERS = ["host/cache_manager.hpp", "host/step_builder.hpp", "host/scheduler.hpp", "host/safetensors.hpp"]


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++)")


def build_host(verbose: bool = False) -> str:
    """The host library (cache manager, step builder): plain C++, no CUDA needed."""
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]
    h = hashlib.sha256()
    for n in HOST_SOURCES + HOST_HEADERS:
        with open(os.path.join(CSRC, n), "rb") as f:
            h.update(n.encode())
            h.update(f.read())
    h.update(" ".join(flags).encode())
    tag = h.hexdigest()[:16]
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"liballpaca_host.{tag}.so")
    if os.path.isfile(lib):
        return lib
    with _Progress("allpaca_host (" + ", ".join(HOST_SOURCES) + ")"):
        tmp = lib + f".tmp{os.getpid()}"
        log = _run([find_cxx()] + flags + ["-o", tmp] + [os.path.join(CSRC, s) for s in HOST_SOURCES])
        os.replace(tmp, lib)
    if verbose:
        print(log, file=sys.stderr)
    for f in os.listdir(out_dir):
        if f.startswith("liballpaca_host.") and f.endswith(".so") and f != os.path.basename(lib):
            try:
                os.remove(os.path.join(out_dir, f))
            except OSError:
                pass
    return lib


def build_core(verbose: bool = False) -> str:
    return build_library("allpaca_core", CORE_SOURCES, verbose=verbose)


def check_head_dim(head_dim: int) -> None:
    if head_dim <= 0 or head_dim % 16 != 0 or head_dim > 256:
        raise BuildError(
            f"head size {head_dim} is not supported by the attention kernels "
            f"(multiples of 16 up to 256)")


def build_attention(head_dim: int, verbose: bool = False) -> str:
    check_head_dim(head_dim)
    return build_library(f"allpaca_attn{head_dim}", ATTN_SOURCES,
                         defines=[f"AP_HEAD_DIM={head_dim}"], verbose=verbose)


def build_all(head_dims: Sequence[int] = (16, 32, 64, 128), verbose: bool = False) -> Dict[str, str]:
    out = {"host": build_host(verbose), "core": build_core(verbose)}
    for hd in head_dims:
        out[f"attn{hd}"] = build_attention(hd, verbose)
    return out


if __name__ == "__main__":
    v = "-v" in sys.argv
    for k, p in build_all(verbose=v).items():
        print(k, p)
