"""Builds the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each family of kernels is one shared library, compiled by nvcc the first time one of
its functions is needed and kept under ``csrc/_build`` (or, when the package folder
cannot be written, under a per-user folder of the temporary directory).  The file name
carries a hash of the sources and flags, so an edited source is rebuilt and a stale
library is never loaded.  While nvcc runs, a line is printed to standard error now and
then, since a cold build takes from seconds to a minute per family.

There is no fallback: if nvcc is missing or a build fails, ``ExtensionError`` is raised."""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional

from ..errors import ExtensionError

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

# family -> (sources, headers it includes, extra flags, libraries)
FAMILIES: Dict[str, dict] = {
    "elementwise": dict(sources=["elementwise.cu"], headers=["common.cuh"]),
    "gemm_plain": dict(sources=["gemm_plain.cu"], headers=["common.cuh"]),
    "rope": dict(sources=["rope.cu"], headers=["common.cuh"]),
    "attention_generic": dict(sources=["attention_generic.cu"], headers=["common.cuh"]),
    "sampling": dict(sources=["sampling.cu"], headers=["common.cuh"]),
    "gemv": dict(sources=["gemv.cu"], headers=["common.cuh"]),
    "attention_decode": dict(sources=["attention_decode.cu"], headers=["common.cuh", "attention_decode.h"]),
    "attention_prefill": dict(sources=["attention_prefill.cu"], headers=["common.cuh", "mma_tiles.cuh"]),
    "gemm_tc": dict(sources=["gemm_tc.cu"], headers=["common.cuh", "tc_common.cuh"]),
    "attention_prefill_tc": dict(sources=["attention_prefill_tc.cu"], headers=["common.cuh", "tc_common.cuh"]),
    "attention_decode_tc": dict(sources=["attention_decode_tc.cu"], headers=["common.cuh", "mma_tiles.cuh"]),
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


def register_family(name: str, sources: List[str], headers: List[str] = (), flags: List[str] = (),
                    libs: List[str] = ()) -> None:
    FAMILIES[name] = dict(sources=list(sources), headers=list(headers), flags=list(flags), libs=list(libs))


def find_nvcc() -> str:
    for base in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if base and os.path.isfile(os.path.join(base, "bin", "nvcc")):
            return os.path.join(base, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise ExtensionError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                         "the CUDA kernels of libllm_b200 cannot be built and there is no fallback")


_build_dir = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is None:
        with _dir_lock:
            if _build_dir is None:
                _build_dir = _find_build_dir()
    return _build_dir


def _find_build_dir() -> str:
    preferred = os.environ.get("LIBLLM_B200_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return preferred
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"libllm_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _family_hash(name: str) -> str:
    fam = FAMILIES[name]
    h = hashlib.sha1()
    for f in list(fam["sources"]) + list(fam.get("headers", ())):
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + list(fam.get("flags", ())) + list(fam.get("libs", ()))).encode())
    return h.hexdigest()[:12]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libllm_{name}-{_family_hash(name)}.so")


def _say(msg: str) -> None:
    print(f"[libllm_b200] {msg}", file=sys.stderr, flush=True)


def _compile(name: str) -> str:
    out = library_path(name)
    if os.path.isfile(out):
        return out
    fam = FAMILIES[name]
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + COMMON_FLAGS + list(fam.get("flags", ())) + ["-I", HERE, "-o", tmp] \
        + [os.path.join(HERE, s) for s in fam["sources"]] + list(fam.get("libs", ()))
    _say(f"compiling {', '.join(fam['sources'])} for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    while True:
        try:
            text, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _say(f"... still compiling {name} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise ExtensionError(f"nvcc failed for {name} (exit {proc.returncode}):\n{text}")
    os.replace(tmp, out)
    # Libraries of this family built from earlier versions of the sources are of no use any more.
    prefix = f"libllm_{name}-"
    for f in os.listdir(os.path.dirname(out)):
        if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(out):
            try:
                os.unlink(os.path.join(os.path.dirname(out), f))
            except OSError:
                pass
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def ensure_built(names: Optional[Iterable[str]] = None) -> List[str]:
    """Compiles the named families (all by default), several at a time."""
    names = list(names) if names is not None else list(FAMILIES)
    todo = [n for n in names if not os.path.isfile(library_path(n))]
    if todo:
        workers = max(1, min(len(todo), (os.cpu_count() or 2)))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            list(pool.map(_compile, todo))
    return [library_path(n) for n in names]


def load(name: str) -> ctypes.CDLL:
    """The shared library of one family, built first if need be."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            if name not in FAMILIES:
                raise ExtensionError(f"no kernel family named '{name}'")
            path = _compile(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
    return lib
