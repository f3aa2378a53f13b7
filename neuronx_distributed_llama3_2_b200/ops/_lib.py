"""Loader/builder for the in-tree sm_100a kernel library ``libnxd_b200.so``.

The library is plain C-ABI (declarations in ``include/nxd_b200.h``): every entry
point takes raw device pointers, sizes and a ``cudaStream_t`` and returns 0 or a
non-zero error code (``nxd_last_error()`` gives the text).  Python binds it with
``ctypes`` and passes ``tensor.data_ptr()`` plus the current torch stream, so the
kernels run in-order with the rest of the eager program and are CUDA-graph
capturable.

There is no silent fallback on a GPU machine: if CUDA is available but the
library is missing, ``available()`` raises unless ``NXD_ALLOW_TORCH_FALLBACK=1``.
"""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_REPO = os.path.dirname(os.path.dirname(_HERE))
CSRC_DIR = os.path.join(_REPO, "csrc")
INCLUDE_DIR = os.path.join(_REPO, "include")
LIB_PATH = os.environ.get("NXD_B200_LIB") or os.path.join(_HERE, "libnxd_b200.so")   # override: kernel experiments
BUILD_DIR = os.environ.get("NXD_BUILD_DIR") or os.path.join(_REPO, "build", "obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
] + [f for f in os.environ.get("NXD_NVCC_EXTRA", "").split() if f]

# Kernel groups: a model family whose kernels live in a few sources of their own can be served from a small library
# built from just those sources (plus the runtime helpers), so a fresh checkout compiles only what that family needs.
# When the full library is already built it contains every group and is used instead.
GROUPS = {
    "window_moe": ["window_attention.cu", "post_norm.cu", "moe_sparse.cu", "runtime.cu"],
}
# everything a bf16 serving step of the window / sparse-MoE families touches: their own kernels, the GEMM kernels behind
# the linear layers, and the tcgen05 flash attention that the windowed prefill is an instantiation of
GROUPS["window_moe_serving"] = GROUPS["window_moe"] + [
    "gemm_tcgen05.cu", "gemm_smallm.cu", "fused_gemm_ar.cu", "tma_host.cu", "flash_attn_tc.cu", "attn_tc_host.cu"]

# the hybrid families (chunked / latent attention, recurrent matrix memory, dense feed-forward): the attention-over-cache
# kernels, the norm kernels, their own two sources and the GEMM kernels behind the linear layers
GROUPS["hybrid_serving"] = ["window_attention.cu", "post_norm.cu", "latent_attention.cu", "mlstm.cu", "runtime.cu",
                            "gemm_tcgen05.cu", "gemm_smallm.cu", "fused_gemm_ar.cu", "tma_host.cu", "flash_attn_tc.cu",
                            "attn_tc_host.cu"]

# the delta-rule hybrids (gated delta rule, differential window attention, dense and sparse gated feed-forward on a
# gated parallel residual): the attention-over-cache, norm, sparse-MoE and recurrent-output kernels, the recurrence's
# own source and the GEMM kernels behind the linear layers
GROUPS["delta_serving"] = ["window_attention.cu", "post_norm.cu", "moe_sparse.cu", "mlstm.cu", "delta_rule.cu",
                           "runtime.cu", "gemm_tcgen05.cu", "gemm_smallm.cu", "fused_gemm_ar.cu", "tma_host.cu"]

# the retention hybrids (softmax attention with sinks next to fixed-decay linear attention, several residual streams,
# dense and sparse gated feed-forward): attention over the cache, sparse MoE, the head norm / gate of recurrent outputs,
# their own two sources, the GEMM kernels behind the linear layers and the tcgen05 flash attention of sink-free prompts
GROUPS["retention_serving"] = ["window_attention.cu", "moe_sparse.cu", "mlstm.cu", "retention.cu", "hyper_connection.cu",
                               "runtime.cu", "gemm_tcgen05.cu", "gemm_smallm.cu", "fused_gemm_ar.cu", "tma_host.cu",
                               "flash_attn_tc.cu", "attn_tc_host.cu"]

# sources whose fp32 state is carried over thousands of steps: no approximate exp / tanh / division
PRECISE_SOURCES = {"mlstm.cu", "delta_rule.cu", "retention.cu", "hyper_connection.cu"}

_lib: Optional[ctypes.CDLL] = None
_group_libs = {}
_preferred_group: Optional[str] = None
_lock = threading.Lock()


def prefer_group(group: Optional[str]) -> None:
    """A program that serves one family only (a command-line tool) names the kernel group it needs: while the full
    library is not built, every ``lib()`` call is answered from that group's library, so a fresh checkout compiles
    that group and nothing else.  An entry point that the group does not hold falls through to the full library."""
    global _preferred_group
    assert group is None or group in GROUPS, group
    _preferred_group = group


class _GroupLibrary:
    """A group's library that hands every entry point it does not have to the full library (built on that first miss)."""

    def __init__(self, handle: ctypes.CDLL):
        self._handle = handle

    def __getattr__(self, name):
        try:
            fn = getattr(self._handle, name)
        except AttributeError:
            fn = getattr(_full_lib(), name)
        setattr(self, name, fn)
        return fn
launch_count = 0  # number of our kernels' entry points invoked (bench "gpu_launches")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources() -> List[str]:
    return sorted(glob.glob(os.path.join(CSRC_DIR, "*.cu")))


def group_sources(group: str) -> List[str]:
    return [os.path.join(CSRC_DIR, f) for f in GROUPS[group]]


def group_lib_path(group: str) -> str:
    return os.path.join(_HERE, f"libnxd_b200_{group}.so")


def _stale(group: Optional[str] = None) -> bool:
    path = group_lib_path(group) if group else LIB_PATH
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    deps = ((group_sources(group) if group else sources()) + glob.glob(os.path.join(CSRC_DIR, "*.cuh"))
            + glob.glob(os.path.join(INCLUDE_DIR, "*.h")))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, group: Optional[str] = None) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libnxd_b200.so`` in-tree; with ``group`` only that group's
    sources, linked as ``libnxd_b200_<group>.so``.

    Works without a GPU (nvcc cross-compiles).  Per-file objects are cached under
    ``build/obj`` and rebuilt only when the source (or any header) is newer.
    """
    out_path = group_lib_path(group) if group else LIB_PATH
    if not force and not _stale(group):
        return out_path
    os.makedirs(BUILD_DIR, exist_ok=True)
    hdrs = glob.glob(os.path.join(CSRC_DIR, "*.cuh")) + glob.glob(os.path.join(INCLUDE_DIR, "*.h"))
    hdr_time = max([os.path.getmtime(h) for h in hdrs], default=0.0)
    nvcc = _nvcc()
    logs = {}

    def compile_one(src: str) -> str:
        obj = os.path.join(BUILD_DIR, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src)
                and os.path.getmtime(obj) > hdr_time):
            return obj
        flags = [f for f in NVCC_FLAGS if not (f == "--use_fast_math" and os.path.basename(src) in PRECISE_SOURCES)]
        cmd = [nvcc] + flags + ["-I", INCLUDE_DIR, "-I", CSRC_DIR, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        logs[src] = res.stderr
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, group_sources(group) if group else sources()))
    tmp = out_path + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp] + objs + ["-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, out_path)
    if logs:
        with open(os.path.join(BUILD_DIR, f"ptxas_v_{group}.log" if group else "ptxas_v.log"), "w") as f:
            for src, text in logs.items():
                f.write(f"==== {os.path.basename(src)}\n{text}\n")
    if verbose:
        for src, text in logs.items():
            sys.stderr.write(f"==== {src}\n{text}\n")
    return out_path


def lib(group: Optional[str] = None) -> ctypes.CDLL:
    """The kernel library.  ``group``: a library that holds at least that kernel group -- the full one when it is
    loaded or built and current, else the group's own small library (built on first use)."""
    if _lib is not None:
        return _lib
    group = _preferred_group or group
    if group is not None and group in _group_libs:       # already serving from the group's library: no file checks
        return _group_libs[group]
    if group is not None and "NXD_B200_LIB" not in os.environ and _stale():
        with _lock:
            handle = _group_libs.get(group)
            if handle is None:
                try:
                    cdll = ctypes.CDLL(build(group=group))
                    cdll.nxd_last_error.restype = ctypes.c_char_p
                    handle = _GroupLibrary(cdll)
                except OSError:          # a source of the group needs a symbol from outside it: use the full library
                    handle = None
                if handle is not None:
                    _group_libs[group] = handle
        if handle is not None:
            return handle
    return _full_lib()


def _full_lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                build()
            handle = ctypes.CDLL(LIB_PATH)
            handle.nxd_last_error.restype = ctypes.c_char_p
            _lib = handle
    return _lib


def available(group: Optional[str] = None) -> bool:
    """True when our CUDA kernels are usable (a GPU is present and the .so loads)."""
    if not torch.cuda.is_available():
        return False
    if os.environ.get("NXD_FORCE_TORCH", "0") == "1":
        return False
    try:
        lib(group)
        return True
    except Exception as e:
        if os.environ.get("NXD_ALLOW_TORCH_FALLBACK", "0") == "1":
            return False
        raise RuntimeError(
            f"CUDA is available but the sm_100a kernel library could not be loaded from {LIB_PATH}: {e}. "
            "Run `python -c 'import __graft_entry__ as g; g.build()'` (or set NXD_ALLOW_TORCH_FALLBACK=1)."
        ) from e


def kernel_launches() -> int:
    """Kernel launches made by the library in this process so far (counted at every ``<<<>>>`` in csrc/)."""
    total = 0
    for handle in ([_lib] if _lib is not None else []) + [g._handle for g in _group_libs.values()] or [lib()]:
        fn = handle.nxd_kernel_launches
        fn.restype = ctypes.c_ulonglong
        total += int(fn())
    return total


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(code: int, what: str, handle: Optional[ctypes.CDLL] = None) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        msg = (handle or lib()).nxd_last_error()
        raise RuntimeError(f"{what} failed (code {code}): {msg.decode() if msg else ''}")


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())
