"""Compiles the CUDA sources of this folder for sm_100a into shared libraries, on demand.

``core_library()`` builds (or finds up to date) the library of kernels every model needs;
``specialised_library(name, source, defines)`` builds one translation unit with ``-D``
definitions, for kernels that are compiled per head size.  Objects and libraries go to
``_build/`` inside this folder, or, when that is not writable, to a per-user folder under
the system temp directory (``DISPEC_B200_BUILD_DIR`` overrides both).  A content hash of
sources, headers and flags decides whether a library is current; nothing is rebuilt
otherwise.  Progress goes to stderr, one line per file, so that a first call in a fresh
checkout is visibly alive.
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

HERE = os.path.dirname(os.path.abspath(__file__))

CORE_SOURCES = [
    "runtime.cu",
    "elementwise.cu",
    "gemm_simt.cu",
    "gemm_tcgen05.cu",
    "gemm_stream.cu",
    "attn_generic.cu",
    "attn_combine.cu",
    "sampling.cu",
    "random_fill.cu",
    "selftest.cu",
]

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# DISPEC_B200_STAMPS=1: a build of its own (another hash) whose weight-streaming product records
# timestamps at eight points of every CTA's life (measurements only)
if os.environ.get("DISPEC_B200_STAMPS") == "1":
    COMMON_FLAGS = COMMON_FLAGS + ["-DDSP_STAMPS"]

_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[dispec_b200 build] {msg}", file=sys.stderr, flush=True)


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if not cand:
        for root in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
            if root and os.path.exists(os.path.join(root, "bin", "nvcc")):
                cand = os.path.join(root, "bin", "nvcc")
                break
    if not cand:
        raise BuildError("nvcc not found (set NVCC or CUDA_HOME); the kernels cannot be compiled")
    return cand


def build_dir() -> str:
    override = os.environ.get("DISPEC_B200_BUILD_DIR")
    candidates = [override] if override else [os.path.join(HERE, "_build")]
    candidates.append(os.path.join(tempfile.gettempdir(), f"dispec_b200_build_{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {candidates}")


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest(sources: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    for name in sources + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    _say(f"{what} done in {time.time() - t0:.1f}s")


def _build(lib_name: str, sources: list[str], defines: list[str], verbose_ptxas: bool = False) -> str:
    flags = ARCH_FLAGS + COMMON_FLAGS + defines + (["-Xptxas", "-v"] if verbose_ptxas else [])
    digest = _digest(sources, flags)
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"{lib_name}.{digest}.so")
    if os.path.exists(lib):
        return lib
    with _lock:
        if os.path.exists(lib):
            return lib
        nvcc = nvcc_path()
        _say(f"compiling {lib_name} ({len(sources)} file(s)) for sm_100a into {out_dir}")
        objs = []

        def compile_one(src: str) -> str:
            obj = os.path.join(out_dir, f"{lib_name}.{digest}.{os.path.splitext(src)[0]}.o")
            _run([nvcc, "-c", os.path.join(HERE, src), "-o", obj, "-I", HERE] + flags, f"nvcc {src}")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            objs = list(pool.map(compile_one, sources))
        tmp = lib + f".tmp{os.getpid()}"
        _run([nvcc, "-shared", "-o", tmp] + objs + ARCH_FLAGS, f"link {lib_name}")
        os.replace(tmp, lib)
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
        # drop stale builds of the same library
        for f in os.listdir(out_dir):
            if f.startswith(lib_name + ".") and f.endswith(".so") and f != os.path.basename(lib):
                try:
                    os.remove(os.path.join(out_dir, f))
                except OSError:
                    pass
    return lib


def core_library() -> str:
    return _build("libdispec_b200_core", CORE_SOURCES, [])


def specialised_library(name: str, source: str, defines: dict[str, int]) -> str:
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    return _build(f"libdispec_b200_{name}", [source], dflags)


def build_all(head_dims=(16, 32, 64, 128)) -> list[str]:
    """Everything a first call could need, for the head sizes given."""
    libs = [core_library()]
    for d in head_dims:
        libs.append(attention_library(d))
        if d in (64, 128):
            libs.append(prefill_attention_library(d))
    return libs


def attention_library(head_dim: int) -> str:
    return specialised_library(f"attn_mma_d{head_dim}", "attn_mma.cu", {"DSP_HEAD_DIM": head_dim})


def prefill_attention_library(head_dim: int) -> str:
    return specialised_library(f"attn_tcgen05_d{head_dim}", "attn_tcgen05.cu", {"DSP_HEAD_DIM": head_dim})


if __name__ == "__main__":
    for path in build_all():
        print(path)
