"""Builds and loads the CUDA kernel libraries (`csrc/*.cu` -> shared objects) and nothing else.

The kernels are plain CUDA with `extern "C"` launchers; they are compiled with
nvcc for sm_100a and loaded through ctypes, so the build needs neither the
torch headers nor a writable HOME.  The first call compiles what is missing or
out of date (a few files in parallel, a progress line now and then on stderr);
later calls find the library by the hash of its sources and flags.  The kernels every engine needs are one
library ("core"); each optional decode kernel is a library of its own, compiled when an engine first asks for it.

There is no fallback: if the library cannot be built or loaded, every kernel
call raises `KernelLibraryError`.
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

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]
LIB_NAME = "libvelomind_b200_kernels.so"
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


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _nvcc() -> str:
    for cand in (os.environ.get("VELOMIND_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelLibraryError("nvcc not found (looked at $VELOMIND_NVCC, PATH and /usr/local/cuda/bin): "
                             "the kernels cannot be compiled")


def _digest(group: str = "core") -> str:
    h = hashlib.sha256()
    for p in sources(group) + _headers():
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
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
    srcs = sources(group)
    _say(f"compiling {len(srcs)} CUDA file{'s' if len(srcs) > 1 else ''} ({group}) for sm_100a into {bdir} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        objs = [os.path.join(bdir, os.path.basename(s)[:-3] + f".{digest}.o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose_ptxas) for s, o in zip(srcs, objs)]
            for s, fu in zip(srcs, futs):
                fu.result()
                _say(f"compiled {os.path.basename(s)} ({time.time() - t0:.0f} s)")
        tmp_target = target + f".{os.getpid()}.tmp"
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_target, *objs, "-lcudart"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelLibraryError(f"linking {name} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp_target, target)
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
