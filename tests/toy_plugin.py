"""Builds tests/cpp/toy_parts.cu into a plug-in library and loads it beside the library: its parts and architectures
register themselves when it is loaded, through the public header alone."""
import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
_loaded = None


def load(workdir: str):
    """Compile (into `workdir`) and load the plug-in once per process; returns the ctypes handle."""
    global _loaded
    if _loaded is not None:
        return _loaded
    from velomind_b200.kernels import library
    main = library.build()
    library.library()                                   # the library itself first, globally: the plug-in resolves against it
    out = os.path.join(workdir, "libtoy_parts.so")
    bdir = os.path.dirname(main)
    cmd = [library._nvcc(), *library.ARCH_FLAGS, "-std=c++17", "-O2", "-Xcompiler", "-fPIC", "-shared", "-I", library.INCLUDE,
           os.path.join(HERE, "cpp", "toy_parts.cu"), "-o", out, "-L", bdir, "-l:" + os.path.basename(main), "-Xlinker", f"-rpath={bdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the toy plug-in failed:\n" + r.stdout + r.stderr)
    _loaded = ctypes.CDLL(out, mode=ctypes.RTLD_GLOBAL)
    _loaded.toy_parts_registered.restype = ctypes.c_char_p
    return _loaded
