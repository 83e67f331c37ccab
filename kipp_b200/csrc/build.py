"""Builds the CUDA sources of this folder into shared libraries for sm_100a
and loads them with ctypes; the C++ sources under ``host/`` (the host core:
configuration, checkpoints, parts, cache manager, step function, scheduler and
the C interface, ``libkipp_engine.so``) are built with the C++ compiler in the
same way and linked against the CUDA runtime.

Each ``<name>.cu`` becomes ``_build/lib<name>.so`` the first time one of its
kernels is needed, so a run compiles only what its model uses.  A library is
rebuilt when its source, a shared header or the flags change.  While nvcc runs,
a line is printed to stderr every few seconds.  There is no fallback: a missing
compiler or a failed build raises.
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

_HERE = os.path.dirname(os.path.abspath(__file__))
_HEADERS = ("common.cuh",)
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_build_dir: str | None = None


class BuildError(RuntimeError):
    pass


def source_names() -> list[str]:
    return sorted(f[:-3] for f in os.listdir(_HERE) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("KIPP_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (set CUDA_HOME or KIPP_B200_NVCC); the CUDA kernels of "
                     "kipp_b200 cannot be built and there is no fallback")


def build_dir() -> str:
    """In-tree ``_build`` when writable, else a per-user temporary folder."""
    global _build_dir
    if _build_dir is not None:
        return _build_dir
    override = os.environ.get("KIPP_B200_BUILD_DIR")
    cands = [override] if override else [os.path.join(_HERE, "_build")]
    cands.append(os.path.join(tempfile.gettempdir(), f"kipp_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".probe", dir=d)
            os.close(fd)
            os.unlink(probe)
            _build_dir = d
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _local_includes(name: str) -> tuple:
    """Files of this folder that ``<name>.cu`` includes by name (one level)."""
    out = []
    with open(os.path.join(_HERE, name + ".cu"), "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line.startswith('#include "'):
                inc = line.split('"')[1]
                if os.path.isfile(os.path.join(_HERE, inc)) and inc not in _HEADERS:
                    out.append(inc)
    return tuple(sorted(set(out)))


def _digest(name: str, extra_flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in (name + ".cu",) + _HEADERS + _local_includes(name) + tuple(sorted(
            x for x in os.listdir(_HERE) if x.endswith(".cuh") and x not in _HEADERS)):
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + extra_flags).encode())
    return h.hexdigest()


def _extra_flags(name: str) -> list[str]:
    flags: list[str] = []
    path = os.path.join(_HERE, name + ".cu")
    with open(path, "r", encoding="utf-8") as f:
        head = f.read(4096)
    for line in head.splitlines():
        if line.startswith("// nvcc-flags:"):
            flags += line.split(":", 1)[1].split()
    return flags


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"lib{name}.so")


def compile_library(name: str, *, verbose: bool = True, force: bool = False) -> str:
    """Compile ``<name>.cu`` if its library is missing or stale; return the path."""
    src = os.path.join(_HERE, name + ".cu")
    if not os.path.isfile(src):
        raise BuildError(f"no CUDA source {src}")
    out_dir = build_dir()
    so = os.path.join(out_dir, f"lib{name}.so")
    stamp = so + ".sha256"
    extra = _extra_flags(name)
    digest = _digest(name, extra)

    def fresh() -> bool:
        try:
            with open(stamp, "r") as f:
                return os.path.isfile(so) and f.read().strip() == digest
        except OSError:
            return False

    if not force and fresh():
        return so
    lock_path = os.path.join(out_dir, f".{name}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return so
            tmp = f"{so}.{os.getpid()}.tmp"
            cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-I", _HERE, "-o", tmp, src]
            if verbose:
                print(f"[kipp_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                    cwd=out_dir)
            out_chunks: list[str] = []
            reader = threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)
            reader.start()
            while True:
                try:
                    proc.wait(timeout=10)
                    break
                except subprocess.TimeoutExpired:
                    if verbose:
                        print(f"[kipp_b200] still compiling {name}.cu ({time.time() - t0:.0f} s)",
                              file=sys.stderr, flush=True)
            reader.join()
            if proc.returncode != 0:
                try:
                    os.unlink(tmp)
                except OSError:
                    pass
                raise BuildError(f"nvcc failed for {name}.cu:\n{' '.join(cmd)}\n{''.join(out_chunks)}")
            os.replace(tmp, so)
            with open(stamp, "w") as f:
                f.write(digest)
            if verbose:
                print(f"[kipp_b200] built lib{name}.so in {time.time() - t0:.1f} s", file=sys.stderr,
                      flush=True)
            return so
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


# ---------------------------------------------------------------------- the host core
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-Wall"]
ENGINE_LIBRARY = "kipp_engine"
_HOST_SOURCES = ("kipp_engine.cpp", "cache_core.cpp")


def _cxx() -> str:
    for cand in (os.environ.get("KIPP_B200_CXX"), os.environ.get("CXX"), shutil.which("g++"),
                 shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler found (set CXX or KIPP_B200_CXX); the host core of kipp_b200 "
                     "cannot be built and there is no fallback")


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda",
                 os.path.dirname(os.path.dirname(_nvcc()))):
        if cand and os.path.isfile(os.path.join(cand, "include", "cuda_runtime_api.h")):
            return cand
    raise BuildError("the CUDA toolkit's headers were not found (set CUDA_HOME)")


def host_source_names() -> list[str]:
    return [ENGINE_LIBRARY]


def compile_host_library(name: str = ENGINE_LIBRARY, *, verbose: bool = True) -> str:
    """Compile the host core (``host/*.cpp`` with its headers) into
    ``lib<name>.so`` if that is missing or stale."""
    if name != ENGINE_LIBRARY:
        raise BuildError(f"no host library {name!r}")
    host = os.path.join(_HERE, "host")
    out_dir = build_dir()
    so = os.path.join(out_dir, f"lib{name}.so")
    stamp = so + ".sha256"
    cuda = _cuda_home()
    lib_dir = os.path.join(cuda, "lib64")
    link = ["-I", os.path.join(cuda, "include"), "-L", lib_dir, "-lcudart", "-ldl", f"-Wl,-rpath,{lib_dir}"]
    h = hashlib.sha256()
    for f in sorted(os.listdir(host)):
        if f.endswith((".cpp", ".hpp", ".h")):
            with open(os.path.join(host, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(HOST_FLAGS + link).encode())
    digest = h.hexdigest()

    def fresh() -> bool:
        try:
            with open(stamp, "r") as f:
                return os.path.isfile(so) and f.read().strip() == digest
        except OSError:
            return False

    if fresh():
        return so
    with open(os.path.join(out_dir, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return so
            tmp = f"{so}.{os.getpid()}.tmp"
            cmd = [_cxx()] + HOST_FLAGS + ["-o", tmp] + [os.path.join(host, f) for f in _HOST_SOURCES] + link
            if verbose:
                print(f"[kipp_b200] compiling the host core (lib{name}.so) ...", file=sys.stderr, flush=True)
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=out_dir)
            out_chunks: list[str] = []
            reader = threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)
            reader.start()
            while True:
                try:
                    proc.wait(timeout=10)
                    break
                except subprocess.TimeoutExpired:
                    if verbose:
                        print(f"[kipp_b200] still compiling the host core ({time.time() - t0:.0f} s)",
                              file=sys.stderr, flush=True)
            reader.join()
            if proc.returncode != 0:
                try:
                    os.unlink(tmp)
                except OSError:
                    pass
                raise BuildError(f"the C++ compiler failed for the host core:\n{' '.join(cmd)}\n{''.join(out_chunks)}")
            os.replace(tmp, so)
            with open(stamp, "w") as f:
                f.write(digest)
            if verbose:
                print(f"[kipp_b200] built lib{name}.so in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
            return so
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_resolver_keepalive = None
_resolved_paths: dict = {}


def load_host_library(name: str = ENGINE_LIBRARY) -> ctypes.CDLL:
    """The host core, built at first use.  It finds the kernel libraries through
    a resolver that compiles each of them when a model first needs it."""
    global _resolver_keepalive
    key = "host/" + name
    with _lock:
        lib = _loaded.get(key)
        if lib is not None:
            return lib
    path = compile_host_library(name)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(path)

            @ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_char_p)
            def resolve(kernel_library):
                # returns the address of a path that stays alive in _resolved_paths
                try:
                    text = kernel_library.decode()
                    if text not in _resolved_paths:
                        _resolved_paths[text] = ctypes.create_string_buffer(compile_library(text).encode())
                    return ctypes.addressof(_resolved_paths[text])
                except Exception as e:          # the core reports the missing library
                    print(f"[kipp_b200] {e}", file=sys.stderr, flush=True)
                    return None

            lib.kipp_set_library_resolver.argtypes = [ctypes.c_void_p]
            lib.kipp_set_library_resolver.restype = None
            lib.kipp_set_library_resolver(ctypes.cast(resolve, ctypes.c_void_p))
            _resolver_keepalive = resolve
            _loaded[key] = lib
        return lib


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(compile_library(name))
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True, jobs: int | None = None) -> list[str]:
    """Compile every source of this folder (in parallel); used by the build check."""
    from concurrent.futures import ThreadPoolExecutor
    names = source_names()
    jobs = jobs or min(len(names), os.cpu_count() or 1) or 1
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        built = list(pool.map(lambda n: compile_library(n, verbose=verbose), names))
    return built + [compile_host_library(n, verbose=verbose) for n in host_source_names()]
