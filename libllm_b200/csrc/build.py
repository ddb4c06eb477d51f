"""Builds the native code of this package and loads it with ctypes.

Two kinds of things are built, each the first time something needs it:

* the **kernel families**: every ``.cu`` of this folder is one shared library for sm_100a,
  compiled by nvcc; a model compiles the families that its type, head size and grouping use;
* the **host library** ``libllm_b200`` (configuration, weights, cache, step function, generation
  loop, C interface: the ``.cc`` files of the package) and the ``llm`` program, compiled by g++
  and linked against the CUDA runtime.

Everything lies under ``csrc/_build`` (or, when the package folder cannot be written, under a
per-user folder of the temporary directory).  File names carry a hash of their sources and flags,
so an edited source is rebuilt and a stale library is never loaded; ``kernels.manifest`` in the
same folder tells the host library (and the ``llm`` program, which has no Python around it) where
each family lies.  While a compiler runs, a line is printed to standard error now and then.

There is no fallback: if a compiler is missing or a build fails, ``ExtensionError`` is raised.

    python -m libllm_b200.csrc.build [family ...]      build kernel families (all by default), the
                                                       host library and the llm program
    python -m libllm_b200.csrc.build --for-model DIR [--dtype bfloat16]
                                                       build what that model needs
    python -m libllm_b200.csrc.build --print-cli       print the path of the llm program"""
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
PACKAGE = os.path.dirname(HERE)
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
    "gemm_chain": dict(sources=["gemm_chain.cu"], headers=["common.cuh", "tc_common.cuh"]),
    "attention_prefill_tc": dict(sources=["attention_prefill_tc.cu"], headers=["common.cuh", "tc_common.cuh"]),
    "attention_decode_tc": dict(sources=["attention_decode_tc.cu"], headers=["common.cuh", "mma_tiles.cuh"]),
}

# The host library: every .cc of the package but the command line's main.
HOST_FOLDERS = ["util", "config", "weights", "parts", "cache", "engine", "sampling", "capi", "csrc", "include"]
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-parameter"]
CLI_SOURCE = os.path.join("cli", "llm_main.cc")

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


def register_family(name: str, sources: List[str], headers: List[str] = (), flags: List[str] = (),
                    libs: List[str] = ()) -> None:
    FAMILIES[name] = dict(sources=list(sources), headers=list(headers), flags=list(flags), libs=list(libs))


def cuda_home() -> str:
    for base in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if base and os.path.isfile(os.path.join(base, "bin", "nvcc")):
            return base
    found = shutil.which("nvcc")
    if found:
        return os.path.dirname(os.path.dirname(os.path.realpath(found)))
    raise ExtensionError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                         "the native code of libllm_b200 cannot be built and there is no fallback")


def find_nvcc() -> str:
    return os.path.join(cuda_home(), "bin", "nvcc")


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


def _say(msg: str) -> None:
    print(f"[libllm_b200] {msg}", file=sys.stderr, flush=True)


def _run(cmd: List[str], what: str) -> None:
    """Runs a compiler; says every 15 s that it is still at it; raises with its output on failure."""
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    while True:
        try:
            text, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _say(f"... still compiling {what} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        raise ExtensionError(f"the build of {what} failed (exit {proc.returncode}):\n{text}")


def _remove_older(prefix: str, keep: str, suffixes=(".so", "")) -> None:
    folder = os.path.dirname(keep)
    for f in os.listdir(folder):
        if f.startswith(prefix) and f != os.path.basename(keep) and not f.endswith(".tmp") \
                and os.path.isfile(os.path.join(folder, f)):
            try:
                os.unlink(os.path.join(folder, f))
            except OSError:
                pass


# ---------------------------------------------------------------- kernel families
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


def _compile(name: str) -> str:
    out = library_path(name)
    if os.path.isfile(out):
        return out
    fam = FAMILIES[name]
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [find_nvcc()] + ARCH_FLAGS + COMMON_FLAGS + list(fam.get("flags", ())) + ["-I", HERE, "-o", tmp] \
        + [os.path.join(HERE, s) for s in fam["sources"]] + list(fam.get("libs", ()))
    _say(f"compiling {', '.join(fam['sources'])} for sm_100a ...")
    t0 = time.time()
    try:
        _run(cmd, name)
    except ExtensionError:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise
    os.replace(tmp, out)
    _remove_older(f"libllm_{name}-", out)      # built from earlier versions of the sources
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def write_manifest() -> str:
    """``kernels.manifest``: a line "family file" for every family that is built, read by the host
    library when nobody tells it where a family lies (the ``llm`` program)."""
    path = os.path.join(build_dir(), "kernels.manifest")
    lines = [f"{n} {os.path.basename(library_path(n))}\n" for n in sorted(FAMILIES) if os.path.isfile(library_path(n))]
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        f.writelines(lines)
    os.replace(tmp, path)
    return path


def ensure_built(names: Optional[Iterable[str]] = None) -> List[str]:
    """Compiles the named families (all by default), several at a time."""
    names = list(names) if names is not None else list(FAMILIES)
    for n in names:
        if n not in FAMILIES:
            raise ExtensionError(f"no kernel family named '{n}'")
    todo = [n for n in names if not os.path.isfile(library_path(n))]
    if todo:
        workers = max(1, min(len(todo), (os.cpu_count() or 2)))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            list(pool.map(_compile, todo))
        write_manifest()
    elif not os.path.isfile(os.path.join(build_dir(), "kernels.manifest")):
        write_manifest()
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
            fresh = not os.path.isfile(library_path(name))
            path = _compile(name)
            if fresh:
                write_manifest()
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
    return lib


# ---------------------------------------------------------------- the host library and the llm program
def host_sources() -> List[str]:
    out = []
    for folder in HOST_FOLDERS:
        d = os.path.join(PACKAGE, folder)
        if os.path.isdir(d):
            out += [os.path.join(folder, f) for f in sorted(os.listdir(d)) if f.endswith(".cc")]
    return out


def _host_headers() -> List[str]:
    out = []
    for folder in HOST_FOLDERS:
        d = os.path.join(PACKAGE, folder)
        if os.path.isdir(d):
            out += [os.path.join(folder, f) for f in sorted(os.listdir(d)) if f.endswith(".h")]
    return out


def _host_hash(extra: Iterable[str] = ()) -> str:
    h = hashlib.sha1()
    for f in host_sources() + _host_headers() + list(extra):
        with open(os.path.join(PACKAGE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()[:12]


def host_library_path() -> str:
    return os.path.join(build_dir(), f"libllm_b200-{_host_hash()}.so")


def cli_path() -> str:
    return os.path.join(build_dir(), f"llm-{_host_hash([CLI_SOURCE])}")


def _gxx() -> str:
    found = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not found:
        raise ExtensionError("no C++ compiler found (g++); the host library of libllm_b200 cannot be built")
    return found


def _host_objects() -> List[str]:
    """Compiles the host sources (several at a time) into a folder named by their hash."""
    obj_dir = os.path.join(build_dir(), f"host-{_host_hash()}")
    os.makedirs(obj_dir, exist_ok=True)
    cuda = cuda_home()
    jobs = []
    for src in host_sources():
        obj = os.path.join(obj_dir, src.replace(os.sep, "_")[:-3] + ".o")
        if not os.path.isfile(obj):
            jobs.append((src, obj))

    def one(job):
        src, obj = job
        tmp = f"{obj}.{os.getpid()}.{threading.get_ident()}.tmp"
        _run([_gxx()] + HOST_FLAGS + ["-I", PACKAGE, "-I", os.path.dirname(PACKAGE), "-I", os.path.join(cuda, "include"),
                                      "-c", os.path.join(PACKAGE, src), "-o", tmp], src)
        os.replace(tmp, obj)

    if jobs:
        _say(f"compiling the host library ({len(jobs)} files) ...")
        with concurrent.futures.ThreadPoolExecutor(max(1, min(len(jobs), os.cpu_count() or 2))) as pool:
            list(pool.map(one, jobs))
    return [os.path.join(obj_dir, s.replace(os.sep, "_")[:-3] + ".o") for s in host_sources()]


def _link_flags() -> List[str]:
    return ["-L", os.path.join(cuda_home(), "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]


def build_host() -> str:
    out = host_library_path()
    if os.path.isfile(out):
        return out
    t0 = time.time()
    objs = _host_objects()
    tmp = f"{out}.{os.getpid()}.tmp"
    _run([_gxx(), "-shared", "-o", tmp] + objs + _link_flags(), "libllm_b200")
    os.replace(tmp, out)
    _remove_older("libllm_b200-", out)
    for f in os.listdir(build_dir()):          # object folders of earlier versions
        if f.startswith("host-") and f != f"host-{_host_hash()}":
            shutil.rmtree(os.path.join(build_dir(), f), ignore_errors=True)
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def build_cli() -> str:
    """The ``llm`` program: the host library's objects and its own main in one executable."""
    out = cli_path()
    if os.path.isfile(out):
        return out
    objs = _host_objects()
    tmp = f"{out}.{os.getpid()}.tmp"
    _run([_gxx()] + HOST_FLAGS + ["-I", PACKAGE, "-I", os.path.dirname(PACKAGE), "-o", tmp, os.path.join(PACKAGE, CLI_SOURCE)]
         + objs + ["-rdynamic"] + _link_flags(), "llm")
    os.replace(tmp, out)
    _remove_older("llm-", out)
    return out


_host = None


def load_host() -> ctypes.CDLL:
    """The host library, built first if need be."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                path = build_host()
                try:
                    _host = ctypes.CDLL(path)
                except OSError as e:
                    raise ExtensionError(f"cannot load {path}: {e}") from None
    return _host


# ---------------------------------------------------------------- command line
def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="python -m libllm_b200.csrc.build", description=__doc__.split("\n\n")[0])
    ap.add_argument("families", nargs="*", help="kernel families to build (default: all)")
    ap.add_argument("--for-model", default=None, help="build what the model in this folder needs")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--print-cli", action="store_true", help="build the llm program and print its path")
    args = ap.parse_args(argv)
    if args.for_model:
        from .. import _lib
        fams = _lib.kernel_families_for(args.for_model, args.dtype)
        ensure_built(fams)
    elif not args.print_cli or args.families:
        ensure_built(args.families or None)
    build_host()
    exe = build_cli()
    write_manifest()
    if args.print_cli:
        print(exe)
    return 0


if __name__ == "__main__":
    try:
        sys.exit(main())
    except ExtensionError as e:
        print(f"libllm_b200: {e}", file=sys.stderr)
        sys.exit(1)
