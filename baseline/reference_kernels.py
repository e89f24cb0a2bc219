"""The reference's own CUDA kernels (its ``cuda/src/kernels.cu``, compiled unchanged) behind ctypes.

The reference engine is a Rust workspace and cannot be built where there is no cargo; its
CUDA kernel file is plain CUDA C++ with a flat C interface
(cuda/include/allpaca_cuda_kernels.h:88-192) and compiles with nvcc alone.  This module
builds it into ``baseline/_ref/liballpaca_cuda_ref.so`` with the reference's own flags
(``-O2 -std=c++17``, crates/allpaca-cuda/build.rs:346-358; the architecture is sm_100a, the one
its ``ALLPACA_CUDA_ARCH`` override would give) and wraps the entry points this engine has a
counterpart for.  Nothing of it is on the product path: tests use it as an oracle that is
not this repository's reading of the formulas, and the kernel benchmark times it.

Every kernel of the reference is 32-bit float.  Its attention kernels keep a carry stack that
traps beyond 2^16 chunks of 128 keys (cuda/src/kernels.cu:1594-1600, :1726-1728); callers here
stay at a few thousand keys.

    python baseline/reference_kernels.py          # build (needs the reference's source and nvcc)
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
from ctypes import c_float, c_int32, c_void_p, POINTER
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "liballpaca_cuda_ref.so")
FLAGS = ["-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-w"]


def reference_dir() -> Optional[str]:
    """Where the reference's source tree is: ``$ALLPACA_REFERENCE_DIR``, or ``reference`` beside
    this repository."""
    for cand in (os.environ.get("ALLPACA_REFERENCE_DIR"), os.path.join(os.path.dirname(HERE), "..", "reference")):
        if cand and os.path.isfile(os.path.join(cand, "cuda", "src", "kernels.cu")):
            return os.path.abspath(cand)
    return None


def build(force: bool = False) -> Optional[str]:
    """Compile the reference's kernel file as it is; returns the library's path, or None (with
    the reason on standard error) when the source or nvcc is missing."""
    if os.path.isfile(LIB_PATH) and not force:
        return LIB_PATH
    ref = reference_dir()
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if ref is None or not os.path.isfile(nvcc):
        print("[reference kernels] not built: " + ("the reference's source tree was not found"
              if ref is None else "nvcc was not found"), file=sys.stderr)
        return None
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    tmp = LIB_PATH + f".tmp{os.getpid()}"
    cmd = [nvcc] + FLAGS + ["-I", os.path.join(ref, "cuda", "include"), "-o", tmp,
                            os.path.join(ref, "cuda", "src", "kernels.cu")]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        print("[reference kernels] nvcc failed:\n" + p.stdout[-2000:], file=sys.stderr)
        return None
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


_P, _I, _F = c_void_p, c_int32, c_float
_SIGNATURES = {
    "allpaca_cuda_gemm_nt": [_P, _P, _P, _I, _I, _I, _P],
    "allpaca_cuda_residual_add": [_P, _P, _P, _I, _P],
    "allpaca_cuda_rmsnorm_rows": [_P, _P, _P, _I, _I, _F, _P],
    "allpaca_cuda_silu_mul": [_P, _P, _P, _I, _P],
    "allpaca_cuda_embed_gather": [_P, _I, _P, _I, _P],
    "allpaca_cuda_rope_qk_rows": [_P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P],
    "allpaca_cuda_rope_imrope_qk": [_P, _P, _I, _I, _I, _I, _I, _F, POINTER(c_int32), _P],
    "allpaca_cuda_attention": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
}


class ReferenceKernels:
    """Thin calls on contiguous float32 CUDA tensors; every call checks the status code."""

    def __init__(self, path: str):
        self.lib = ctypes.CDLL(path)
        for name, args in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = args
            fn.restype = c_int32
        self._no_sections = (c_int32 * 4)(0, 0, 0, 0)

    @staticmethod
    def _stream():
        import torch
        return torch.cuda.current_stream().cuda_stream

    @staticmethod
    def _f32(*tensors):
        import torch
        for t in tensors:
            if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
                raise ValueError("the reference's kernels take contiguous float32 CUDA tensors")

    def _call(self, name, *args):
        rc = getattr(self.lib, name)(*args, self._stream())
        if rc != 0:
            raise RuntimeError(f"{name} returned status {rc}")

    def gemm_nt(self, a, w, out):
        """``out[m,n] = a[m,k] w[n,k]^T`` (cuda/src/kernels.cu:431-459)."""
        self._f32(a, w, out)
        m, k = a.shape
        self._call("allpaca_cuda_gemm_nt", a.data_ptr(), w.data_ptr(), out.data_ptr(), m, w.shape[0], k)

    def residual_add(self, x, y, out):
        self._f32(x, y, out)
        self._call("allpaca_cuda_residual_add", x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel())

    def rmsnorm_rows(self, x, w, out, eps):
        self._f32(x, w, out)
        self._call("allpaca_cuda_rmsnorm_rows", x.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                   float(eps))

    def silu_mul(self, gate, up, out):
        self._f32(gate, up, out)
        self._call("allpaca_cuda_silu_mul", gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel())

    def embed_gather(self, table, token, out):
        self._f32(table, out)
        self._call("allpaca_cuda_embed_gather", table.data_ptr(), int(token), out.data_ptr(), table.shape[1])

    def rope_adjacent(self, q, k, start_pos, theta):
        """Pairs ``(2i, 2i+1)`` on ``q [T, heads, hd]`` and ``k [T, kv_heads, hd]`` in place, row ``t`` at
        position ``start_pos + t`` (cuda/src/kernels.cu:1244-1281)."""
        self._f32(q, k)
        T, nq, hd = q.shape
        self._call("allpaca_cuda_rope_qk_rows", q.data_ptr(), k.data_ptr(), T, nq, k.shape[1], hd, nq * hd,
                   k.shape[1] * hd, int(start_pos), float(theta))

    def rope_half_split(self, q, k, start_pos, theta):
        """Pairs ``(i, i + hd/2)`` over the whole head, one launch per row: the reference's
        partial-rotation kernel with every dimension rotated and no sections
        (cuda/src/kernels.cu:1287-1362)."""
        self._f32(q, k)
        T, nq, hd = q.shape
        for t in range(T):
            self._call("allpaca_cuda_rope_imrope_qk", q[t].data_ptr(), k[t].data_ptr(), nq, k.shape[1], hd, hd,
                       int(start_pos) + t, float(theta), self._no_sections)

    def attention(self, q, k, v, out, causal=True):
        """``q [n_q, heads, hd]``, ``k, v [n_kv, kv_heads, hd]``; causal rows are bottom-right aligned
        (cuda/src/kernels.cu:2198-2206)."""
        self._f32(q, k, v, out)
        n_q, nh, hd = q.shape
        self._call("allpaca_cuda_attention", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), n_q,
                   k.shape[0], nh, k.shape[1], hd, 1 if causal else 0)


_loaded: Optional[ReferenceKernels] = None


def load(build_if_missing: bool = True) -> Optional[ReferenceKernels]:
    """The compiled reference kernels, or None when they are not here and cannot be built."""
    global _loaded
    if _loaded is None:
        path = LIB_PATH if os.path.isfile(LIB_PATH) else (build() if build_if_missing else None)
        if path is None:
            return None
        _loaded = ReferenceKernels(path)
    return _loaded


if __name__ == "__main__":
    out = build(force="--force" in sys.argv)
    print(out or "not built")
    sys.exit(0 if out else 1)
