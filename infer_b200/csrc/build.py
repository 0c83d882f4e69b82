"""Compiles the CUDA sources of this package for sm_100a with nvcc and loads them through ctypes.

Each module is one ``.cu`` file compiled into one shared library that exports a C ABI.  Libraries
are built on first use, into ``_build/`` beside the sources (or a per-user temporary folder when
the package is not writable), and are named after a hash of their sources and flags, so an edited
source never meets a stale binary.  While nvcc runs, a progress line is printed every few seconds.
Nothing here needs a GPU: the same call cross-compiles on a machine without one.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Mapping, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]

# module name -> source file; headers that every module depends on
MODULES: Dict[str, str] = {
    "plain": "plain_ops.cu",
    "gemvb": "gemv_bulk.cu",
    "gemm": "gemm_tcgen05.cu",
    "attn": "attention_fast.cu",
    "attn_tc": "attention_tc.cu",
    "capi": "capi.cpp",          # host code only: the C handle API over the engine (needs the interpreter's headers)
}
HEADERS = ["common.cuh", "gemm_static.h", "tma_map.cuh"]
# modules that are compiled per model size: the variant that build_all() makes (others are built at first use)
DEFAULT_DEFINES = {"attn": {"IB_HEAD_DIM": 128}, "attn_tc": {"IB_HEAD_DIM": 128}}


class BuildError(RuntimeError):
    pass


def _module_flags(module: str):
    """Extra compiler flags of a module."""
    if module == "capi":
        import sysconfig
        return ["-I", sysconfig.get_paths()["include"]]
    return []


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the CUDA kernels of infer_b200 cannot be built and there is no fallback")


_BUILD_DIR = None
_BUILD_DIR_LOCK = threading.Lock()


def _build_dir() -> str:
    global _BUILD_DIR
    with _BUILD_DIR_LOCK:
        if _BUILD_DIR is None:
            _BUILD_DIR = _find_build_dir()
        return _BUILD_DIR


def _find_build_dir() -> str:
    env = os.environ.get("INFER_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"infer_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _digest(module: str, defines: Mapping[str, object]) -> str:
    h = hashlib.sha256()
    for fn in [MODULES[module]] + HEADERS:
        with open(os.path.join(HERE, fn), "rb") as f:
            h.update(fn.encode() + b"\0" + f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(repr(sorted(defines.items())).encode())
    return h.hexdigest()[:16]


def library_path(module: str, defines: Optional[Mapping[str, object]] = None) -> str:
    defines = dict(defines or {})
    tag = "".join(f"_{k}{v}" for k, v in sorted(defines.items()))
    return os.path.join(_build_dir(), f"libib_{module}{tag}_{_digest(module, defines)}.so")


def _say(msg: str) -> None:
    print(f"[infer_b200] {msg}", file=sys.stderr, flush=True)


def compile_module(module: str, defines: Optional[Mapping[str, object]] = None, verbose: bool = False) -> str:
    """Builds one module if its library is not there yet; returns the library's path."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module {module!r}")
    defines = dict(defines or {})
    out = library_path(module, defines)
    if os.path.isfile(out):
        return out
    nvcc = _find_nvcc()
    lock_path = out + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out):
                return out
            tmp = f"{out}.{os.getpid()}.tmp"
            cmd = [nvcc] + NVCC_FLAGS + _module_flags(module) + [f"-D{k}={v}" for k, v in sorted(defines.items())] + \
                  ["-I", HERE, "-o", tmp, os.path.join(HERE, MODULES[module])]
            _say(f"compiling {MODULES[module]} for sm_100a (first use; this happens once) ...")
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                    cwd=_build_dir())
            done = threading.Event()

            def ticker():
                while not done.wait(10.0):
                    _say(f"  still compiling {MODULES[module]} ({time.time() - t0:.0f} s)")
            th = threading.Thread(target=ticker, daemon=True)
            th.start()
            log, _ = proc.communicate()
            done.set()
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise BuildError(f"nvcc failed for {MODULES[module]}:\n{' '.join(cmd)}\n{log}")
            with open(out + ".log", "w") as f:
                f.write(" ".join(cmd) + "\n" + log)
            os.replace(tmp, out)
            _say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s")
            if verbose:
                print(log)
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            try:
                os.remove(lock_path)
            except OSError:
                pass


_LOADED: Dict[str, ctypes.CDLL] = {}


def load_module(module: str, defines: Optional[Mapping[str, object]] = None) -> ctypes.CDLL:
    """The module's library, compiled if need be and loaded once per process."""
    path = compile_module(module, defines)
    lib = _LOADED.get(path)
    if lib is None:
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
        if hasattr(lib, "ib_last_error"):                            # (the kernel libraries; the C handle API has its own)
            lib.ib_last_error.restype = ctypes.c_char_p
            if os.environ.get("INFER_B200_PDL", "1") == "0":
                lib.ib_set_pdl(0)       # launch every kernel fully serialised (for comparisons)
        _LOADED[path] = lib
    return lib


def build_all(modules: Optional[Sequence[str]] = None, verbose: bool = False) -> Dict[str, str]:
    """Compiles every module (in parallel); used by the build check and before GPU runs."""
    from concurrent.futures import ThreadPoolExecutor
    names = [m for m in (modules or MODULES) if os.path.isfile(os.path.join(HERE, MODULES[m]))]
    jobs = [(m, DEFAULT_DEFINES.get(m)) for m in names]
    with ThreadPoolExecutor(max_workers=min(8, len(jobs) or 1)) as pool:
        paths = list(pool.map(lambda j: compile_module(j[0], j[1], verbose), jobs))
    return dict(zip(names, paths))
