"""Builds and loads the CUDA kernel libraries, one shared object per kernel family.

Each family is one `.cu` file under `csrc/`, compiled by nvcc for sm_100a only into
`<package>/_build/<family>-<hash>.so` and opened with ctypes. The hash covers the sources, the
shared headers and the flags, so a stale object is never loaded. A family is built at the
first call that needs it: a float32 run never compiles the tensor-core files. While nvcc
runs, a line is printed every few seconds. There is no fallback: if a library cannot be
built or loaded, the call raises `KernelBuildError`.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_CSRC = os.path.join(_PKG, "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]

# family -> (source file, extra nvcc flags, extra link flags)
FAMILIES: Dict[str, tuple] = {
    "elementwise": ("elementwise.cu", [], []),
    "attention_simt": ("attention_simt.cu", [], []),
    "attention_decode": ("attention_decode.cu", [], []),
    "attention_decode_mma": ("attention_decode_mma.cu", [], []),
    "attention_prefill_tc": ("attention_prefill_tc.cu", [], []),
    "gemm_simt": ("gemm_simt.cu", [], []),
    "gemm_skinny": ("gemm_skinny.cu", [], []),
    "gemm_tc": ("gemm_tc.cu", [], []),
    "gemm_stream": ("gemm_stream.cu", [], []),
    "gemm_fused_decode": ("gemm_fused_decode.cu", [], []),
    "sampling": ("sampling.cu", [], []),
}


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def register_family(name: str, source: str, nvcc_flags: Optional[List[str]] = None,
                    link_flags: Optional[List[str]] = None) -> None:
    FAMILIES[name] = (source, list(nvcc_flags or []), list(link_flags or []))


def _nvcc() -> str:
    for cand in (os.environ.get("LLMIE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (PATH, /usr/local/cuda/bin, $LLMIE_NVCC): the CUDA kernels of this "
                           "library cannot be built, and there is no fallback path")


def _headers() -> List[str]:
    return sorted(os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith((".cuh", ".h")))


def _digest(source: str, flags: List[str]) -> str:
    h = hashlib.sha256()
    for path in [source] + _headers():
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode())
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + flags).encode())
    return h.hexdigest()[:16]


def build_dir() -> str:
    """`<package>/_build` when it can be written, else a per-user folder under the temp dir."""
    override = os.environ.get("LLMIE_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(_PKG, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"llm_infer_engine_b200_build_{os.getuid()}"))
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
    raise KernelBuildError(f"no writable build folder among {candidates}")


def _search_dirs() -> List[str]:
    dirs = []
    if os.environ.get("LLMIE_BUILD_DIR"):
        dirs.append(os.environ["LLMIE_BUILD_DIR"])
    dirs.append(os.path.join(_PKG, "_build"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"llm_infer_engine_b200_build_{os.getuid()}"))
    return dirs


def library_path(family: str, must_exist: bool = False) -> Optional[str]:
    src, flags, link = FAMILIES[family]
    name = f"{family}-{_digest(os.path.join(_CSRC, src), flags + link)}.so"
    for d in _search_dirs():
        p = os.path.join(d, name)
        if os.path.isfile(p):
            return p
    return None if must_exist else os.path.join(build_dir(), name)


def _compile(family: str, out_path: str, verbose: bool) -> None:
    src, flags, link = FAMILIES[family]
    src_path = os.path.join(_CSRC, src)
    tmp = f"{out_path}.{os.getpid()}.tmp"
    cmd = [_nvcc()] + ARCH_FLAGS + COMMON_FLAGS + flags + ["-I", _CSRC, "-o", tmp, src_path] + link
    env = dict(os.environ)
    env.setdefault("TMPDIR", os.path.dirname(out_path))  # nvcc's intermediates; HOME may be missing
    t0 = time.time()
    print(f"[llm_infer_engine_b200] compiling kernel family '{family}' for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(5.0):
            print(f"[llm_infer_engine_b200]   still compiling '{family}' ({time.time() - t0:.0f}s)",
                  file=sys.stderr, flush=True)

    th = threading.Thread(target=heartbeat, daemon=True)
    th.start()
    try:
        out, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for kernel family '{family}':\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, out_path)
    # objects of older versions of this family's source are never loaded again: drop them
    folder = os.path.dirname(out_path)
    for name in os.listdir(folder):
        if name.startswith(family + "-") and name.endswith(".so") and os.path.join(folder, name) != out_path:
            try:
                os.remove(os.path.join(folder, name))
            except OSError:
                pass
    if verbose and out.strip():
        print(out, file=sys.stderr)
    print(f"[llm_infer_engine_b200] built '{family}' in {time.time() - t0:.1f}s -> {out_path}", file=sys.stderr, flush=True)


def load(family: str) -> ctypes.CDLL:
    """The family's library, built first if no current object exists."""
    lib = _loaded.get(family)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(family)
        if lib is not None:
            return lib
        if family not in FAMILIES:
            raise KernelBuildError(f"unknown kernel family {family!r}")
        path = library_path(family, must_exist=True)
        if path is None:
            path = library_path(family)
            _compile(family, path, verbose=bool(os.environ.get("LLMIE_BUILD_VERBOSE")))
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from e
        _loaded[family] = lib
        return lib


def build_all(verbose: bool = False) -> Dict[str, str]:
    """Compiles every family whose object is missing; returns family -> path."""
    out = {}
    for family in FAMILIES:
        path = library_path(family, must_exist=True)
        if path is None:
            path = library_path(family)
            _compile(family, path, verbose)
        out[family] = path
    return out
