"""Builds and loads the library: the CUDA kernels (`csrc/*.cu`) and the C++ host (`config/`, `weights/`, `parts/`,
`cache/`, `engine/`, `models/`, `text/`, `capi/`, `apps/`) in ONE shared object, plus the two programs.

The kernels are plain CUDA with `extern "C"` launchers, compiled with nvcc for sm_100a; the host is C++17, compiled
with g++.  Neither needs the torch headers nor a writable HOME.  The first call compiles what is missing or out of
date (files in parallel, a progress line now and then on stderr); later calls find the library by the hash of its
sources and flags.  `CMakeLists.txt` at the repository root builds the same targets from the same file lists.

There is no fallback: if the library cannot be built or loaded, every call raises `KernelLibraryError`.
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
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

PACKAGE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PACKAGE, "csrc")
INCLUDE = os.path.join(PACKAGE, "include")
HOST_DIRS = ["config", "weights", "cache", "parts", "engine", "models", "text", "capi", "apps"]
PROGRAMS = {"smollm2_chat": "apps/smollm2_chat_main.cpp", "trace_run": "apps/trace_run_main.cpp"}
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]
LIB_NAME = "libvelomind_b200.so"
# optional kernels, each a library of its own (group name -> source files); everything else is the "core" library
OPTIONAL = {}


class KernelLibraryError(RuntimeError):
    """The CUDA kernel library is missing and could not be built, or failed to load."""


_lock = threading.Lock()
_libs = {}


def groups() -> List[str]:
    return ["core"] + sorted(OPTIONAL)


def sources(group: str = "core") -> List[str]:
    if group in OPTIONAL:
        return [os.path.join(CSRC, f) for f in OPTIONAL[group]]
    if group != "core":
        raise KernelLibraryError(f"no kernel library named {group!r}")
    held_back = {f for fs in OPTIONAL.values() for f in fs}
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu") and f not in held_back)


def lib_name(group: str = "core") -> str:
    return LIB_NAME if group == "core" else f"libvelomind_b200_{group}.so"


def host_sources() -> List[str]:
    """The C++ files of the library itself (the programs' `*_main.cpp` are linked against it, not into it)."""
    out = []
    for d in HOST_DIRS:
        folder = os.path.join(PACKAGE, d)
        if os.path.isdir(folder):
            out += [os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".cpp") and not f.endswith("_main.cpp")]
    return sorted(out)


def _headers() -> List[str]:
    found = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    for base, _, files in os.walk(INCLUDE):
        found += [os.path.join(base, f) for f in files if f.endswith(".h")]
    for d in HOST_DIRS:
        folder = os.path.join(PACKAGE, d)
        if os.path.isdir(folder):
            found += [os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".h") or f.endswith("_main.cpp")]
    return sorted(found)


def _cuda_home() -> str:
    return os.path.dirname(os.path.dirname(_nvcc()))


def _nvcc() -> str:
    for cand in (os.environ.get("VELOMIND_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelLibraryError("nvcc not found (looked at $VELOMIND_NVCC, PATH and /usr/local/cuda/bin): "
                             "the kernels cannot be compiled")


def _digest(group: str = "core") -> str:
    h = hashlib.sha256()
    for p in sources(group) + (host_sources() if group == "core" else []) + _headers():
        h.update(os.path.relpath(p, PACKAGE).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    """In-tree `csrc/_build` if it can be written, else $VELOMIND_B200_BUILD_DIR, else a per-user temp folder."""
    env = os.environ.get("VELOMIND_B200_BUILD_DIR")
    if env and _writable_dir(env):
        return env
    intree = os.path.join(CSRC, "_build")
    if _writable_dir(intree):
        return intree
    tmp = os.path.join(tempfile.gettempdir(), f"velomind_b200_build_{os.getuid()}")
    if _writable_dir(tmp):
        return tmp
    raise KernelLibraryError(f"no writable folder for the kernel build (tried {intree} and {tmp})")


def _say(msg: str) -> None:
    print(f"[velomind_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, verbose_ptxas: bool) -> None:
    if src.endswith(".cpp"):
        cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
        cmd = [cxx, *CXX_FLAGS, "-I", INCLUDE, "-I", os.path.join(_cuda_home(), "include"), "-c", src, "-o", obj]
        verbose_ptxas = False
    else:
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelLibraryError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
    if verbose_ptxas:
        with open(obj + ".ptxas.txt", "w") as f:
            f.write(r.stderr)


def build(force: bool = False, verbose_ptxas: bool = False, group: str = "core") -> str:
    """Compile the library `group` if its sources changed; return the path of the shared object."""
    bdir = build_dir()
    digest = _digest(group)
    name = lib_name(group)
    target = os.path.join(bdir, name)
    stamp = os.path.join(bdir, "sources.sha" if group == "core" else f"sources.{group}.sha")
    if not force and os.path.isfile(target) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return target
    nvcc = _nvcc()
    srcs = sources(group) + (host_sources() if group == "core" else [])
    _say(f"compiling {len(sources(group))} CUDA files for sm_100a and {len(srcs) - len(sources(group))} C++ files into {bdir} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        objs = [os.path.join(bdir, os.path.relpath(s, PACKAGE).replace(os.sep, "_") + f".{digest}.o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose_ptxas) for s, o in zip(srcs, objs)]
            for s, fu in zip(srcs, futs):
                fu.result()
                _say(f"compiled {os.path.basename(s)} ({time.time() - t0:.0f} s)")
        tmp_target = target + f".{os.getpid()}.tmp"
        lib64 = os.path.join(_cuda_home(), "lib64")
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_target, *objs, "-L", lib64, "-lcublas", "-lpthread",
                            "-Xlinker", f"-rpath={lib64}"], capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelLibraryError(f"linking {name} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp_target, target)
        if group == "core":
            cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
            for prog, main in PROGRAMS.items():
                tmp_prog = os.path.join(bdir, f"{prog}.{os.getpid()}.tmp")
                r = subprocess.run([cxx, *CXX_FLAGS, "-I", INCLUDE, "-I", os.path.join(_cuda_home(), "include"), os.path.join(PACKAGE, main),
                                    "-o", tmp_prog, "-L", bdir, "-l:" + name, "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{lib64}"],
                                   capture_output=True, text=True)
                if r.returncode != 0:
                    raise KernelLibraryError(f"linking {prog} failed:\n{r.stdout}\n{r.stderr}")
                os.replace(tmp_prog, os.path.join(bdir, prog))
        with open(stamp, "w") as f:
            f.write(digest)
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
    finally:
        done.set()
    _say(f"kernel library {name} ready ({time.time() - t0:.0f} s)")
    return target


def program(name: str) -> str:
    """The path of a built program (`smollm2_chat`, `trace_run`); builds the library first if need be."""
    if name not in PROGRAMS:
        raise KernelLibraryError(f"no program named {name!r}")
    build()
    return os.path.join(build_dir(), name)


def library(group: str = "core") -> ctypes.CDLL:
    """The loaded kernel library `group`; built at the first call if need be.  The optional libraries use symbols
    of the core library, which is therefore loaded first and globally."""
    lib = _libs.get(group)
    if lib is not None:
        return lib
    if group != "core":
        library("core")
    with _lock:
        if group not in _libs:
            path = build(group=group)
            try:
                _libs[group] = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            except OSError as e:
                raise KernelLibraryError(f"cannot load {path}: {e}") from None
    return _libs[group]
