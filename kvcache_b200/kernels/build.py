"""Compiles the CUDA sources under `kvcache_b200/csrc` for sm_100a and loads them.

Each `.cu` file becomes one shared library, built the first time one of its
functions is needed and kept beside the sources (`csrc/_build/`), or in a
per-user temporary folder when the package folder cannot be written.  The
library's file name carries a digest of its sources and flags, so an edited
kernel is never served from an old build.  There is no fallback: a missing
compiler or a failed build raises.
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
from typing import Dict, Iterable, List, Optional, Sequence

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"]

# module name -> (source file, headers it includes, extra flags, extra link libraries)
MODULES: Dict[str, dict] = {
    "elementwise": {"src": "elementwise.cu", "deps": ["common.cuh"]},
    "rope_append": {"src": "rope_append.cu", "deps": ["common.cuh"]},
    "attention_generic": {"src": "attention_generic.cu", "deps": ["common.cuh"]},
    "gemm_simt": {"src": "gemm_simt.cu", "deps": ["common.cuh"]},
    "sampling": {"src": "sampling.cu", "deps": ["common.cuh"]},
    "gemm_skinny": {"src": "gemm_skinny.cu", "deps": ["common.cuh"]},
    "gemm_tcgen05": {"src": "gemm_tcgen05.cu", "deps": ["common.cuh", "tc_common.cuh"]},
    # Compiled per head size: variant "d<head_dim>" with -DKVB_HEAD_DIM=<head_dim>.
    "attention_flash": {"src": "attention_flash.cu", "deps": ["common.cuh", "flash_core.cuh", "no_alloc.h", "tc_common.cuh"]},
    "attention_tc": {"src": "attention_tc.cu", "deps": ["common.cuh", "tc_common.cuh"]},
    "gemm_wstream": {"src": "gemm_wstream.cu", "deps": ["common.cuh", "tc_common.cuh"]},
    # What barrier waits, votes, MMA issue and page copies cost on this GPU (python -m kvcache_b200.kernels.primitive_costs).
    "primitive_costs": {"src": "primitive_costs.cu", "deps": ["common.cuh", "tc_common.cuh"]},
    # One wait that cannot end, with a short poll limit: shows that a stalled wait reaches the host as an error bit.
    "wait_probe": {"src": "wait_probe.cu", "deps": ["common.cuh", "tc_common.cuh"], "flags": ["-DKVB_SPIN_LIMIT=4096"]},
}
# Variants that `build_all` makes for modules compiled per size.
DEFAULT_VARIANTS = {"attention_flash": [("d64", ["-DKVB_HEAD_DIM=64"]), ("d128", ["-DKVB_HEAD_DIM=128"])],
                    "attention_tc": [("d64", ["-DKVB_HEAD_DIM=64"]), ("d128", ["-DKVB_HEAD_DIM=128"])]}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _log(message: str) -> None:
    print(f"[kvcache_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (os.environ.get("KVCACHE_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc not found: the CUDA kernels of kvcache_b200 have to be compiled for sm_100a "
                     "(set KVCACHE_B200_NVCC or put nvcc on PATH); there is no fallback path")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}-{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    global _build_dir_cache
    with _dir_lock:
        if _build_dir_cache is None:
            _build_dir_cache = _choose_build_dir()
        return _build_dir_cache


def _choose_build_dir() -> str:
    override = os.environ.get("KVCACHE_B200_BUILD_DIR")
    if override and _writable_dir(override):
        return override
    in_tree = os.path.join(CSRC_DIR, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"kvcache_b200-build-{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"no writable folder for compiled kernels (tried {in_tree} and {fallback})")


def _digest(module: str, extra_flags: Sequence[str]) -> str:
    info = MODULES[module]
    h = hashlib.sha256()
    for name in [info["src"], *info.get("deps", [])]:
        with open(os.path.join(CSRC_DIR, name), "rb") as fh:
            h.update(name.encode())
            h.update(fh.read())
    h.update(" ".join([*ARCH_FLAGS, *BASE_FLAGS, *info.get("flags", []), *extra_flags]).encode())
    return h.hexdigest()[:16]


def library_path(module: str, variant: str = "", extra_flags: Sequence[str] = ()) -> str:
    tag = f"{module}{('-' + variant) if variant else ''}"
    return os.path.join(build_dir(), f"kvb200_{tag}.{_digest(module, extra_flags)}.so")


def _find_built(module: str, variant: str, extra_flags: Sequence[str]) -> Optional[str]:
    """An up-to-date library in any of the places a build may have put it."""
    tag = f"{module}{('-' + variant) if variant else ''}"
    name = f"kvb200_{tag}.{_digest(module, extra_flags)}.so"
    for folder in (os.environ.get("KVCACHE_B200_BUILD_DIR"), os.path.join(CSRC_DIR, "_build"),
                   os.path.join(tempfile.gettempdir(), f"kvcache_b200-build-{os.getuid()}")):
        if folder and os.path.isfile(os.path.join(folder, name)):
            return os.path.join(folder, name)
    return None


def compile_module(module: str, variant: str = "", extra_flags: Sequence[str] = (), force: bool = False) -> str:
    """Builds one module (if its library is missing or stale) and returns the library's path."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module '{module}'")
    if not force:
        found = _find_built(module, variant, extra_flags)
        if found:
            return found
    info = MODULES[module]
    out = library_path(module, variant, extra_flags)
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [find_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *info.get("flags", []), *extra_flags,
           "-I", CSRC_DIR, "-o", tmp, os.path.join(CSRC_DIR, info["src"]), *info.get("libs", [])]
    _log(f"compiling {info['src']}{(' [' + variant + ']') if variant else ''} for sm_100a ...")
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            _log(f"  still compiling {info['src']} ({time.time() - start:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed on {info['src']} (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    _log(f"  built {os.path.basename(out)} in {time.time() - start:.1f} s")
    # Libraries of this module made from older sources are of no use any more.
    prefix = os.path.basename(out).rsplit(".", 2)[0] + "."
    for name in os.listdir(os.path.dirname(out)):
        if name.startswith(prefix) and name.endswith(".so") and name != os.path.basename(out):
            try:
                os.remove(os.path.join(os.path.dirname(out), name))
            except OSError:
                pass
    return out


def load_module(module: str, variant: str = "", extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    key = f"{module}:{variant}"
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_module(module, variant, extra_flags))
            _loaded[key] = lib
        return lib


def build_all(modules: Optional[Iterable[str]] = None, jobs: int = 0) -> List[str]:
    """Compiles every module (in parallel) without loading any; returns the libraries' paths."""
    from concurrent.futures import ThreadPoolExecutor
    names = list(modules) if modules is not None else list(MODULES)
    work = []
    for name in names:
        for variant, flags in DEFAULT_VARIANTS.get(name, [("", [])]):
            work.append((name, variant, tuple(flags)))
    jobs = jobs or min(len(work), os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=max(1, jobs)) as pool:
        return list(pool.map(lambda w: compile_module(*w), work))
