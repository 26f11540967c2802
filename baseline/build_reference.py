"""Builds the UNMODIFIED reference (Aiza-Lee/velo-mind) with its CUDA backend and its own benchmark tool.

    python baseline/build_reference.py [/path/to/reference]     ->  baseline/_ref/benchmark_baseline, baseline/_ref/reference_driver

The reference is a C++23/CMake project; its CMake build of the examples and benchmarks needs git submodules
(sentencepiece, catch2) that are empty in an offline checkout, so the same sources are compiled here directly:
the core (`src/*.cpp`, `src/internal`, `src/cpu`), the CUDA backend (`src/cuda/*.cu`, `src/cuda/ops/*.cu`, with
cuBLAS), the Llama example (`examples/common/llama`, `examples/smollm2`) and `benchmarks/*.cpp`.  Nothing of the
reference is changed or copied; the only added file stands in for the export header that CMake would generate.
The CUDA files are compiled for compute capability 10.0 (the reference's own option
`VELOMIND_CUDA_ARCHITECTURES`, default 89).  Nothing of this repository is linked in.  `reference_driver` is this
repository's own small program (baseline/reference_driver.cpp) that calls the reference's public engine API.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REFERENCE = "/root/reference"
EXE = os.path.join(OUT, "benchmark_baseline")
DRIVER = os.path.join(OUT, "reference_driver")


def sources(ref: str):
    cpp, cu = [], []
    for pat in ("src/*.cpp", "src/internal/*.cpp", "src/internal/registry/*.cpp", "src/cpu/*.cpp", "src/cpu/ops/*.cpp",
                "benchmarks/*.cpp"):
        cpp += sorted(glob.glob(os.path.join(ref, pat)))
    cpp += [os.path.join(ref, p) for p in (
        "examples/common/llama/llama_rope_mask.cpp", "examples/common/llama/llama_graph.cpp",
        "examples/common/llama/llama_engine.cpp", "examples/common/llama/llama_model_finder.cpp",
        "examples/smollm2/config_parser.cpp", "examples/smollm2/model_loader.cpp",
        "examples/smollm2/smollm2_engine.cpp", "examples/smollm2/tokenizer.cpp")]
    for pat in ("src/cuda/*.cu", "src/cuda/ops/*.cu"):
        cu += sorted(glob.glob(os.path.join(ref, pat)))
    return cpp, cu


def build(ref: str = DEFAULT_REFERENCE, force: bool = False) -> str:
    if os.path.isfile(EXE) and os.path.isfile(DRIVER) and not force:
        return EXE
    if not os.path.isdir(os.path.join(ref, "src")):
        raise RuntimeError(f"no checkout of the reference at {ref}")
    obj = os.path.join(OUT, "obj")
    os.makedirs(obj, exist_ok=True)
    with open(os.path.join(OUT, "velomind_core_export.h"), "w") as f:     # stands in for the CMake-generated header
        f.write("#pragma once\n#define VELOMIND_CORE_EXPORT\n#define VELOMIND_CORE_NO_EXPORT\n")
    inc = [f"-I{OUT}", f"-I{ref}/include", f"-I{ref}/src", f"-I{ref}", f"-I{ref}/examples/common/llama",
           f"-I{ref}/examples/smollm2", f"-I{ref}/examples/tinyllama", f"-I{ref}/benchmarks"]
    defs = ["-DVELOMIND_ENABLE_CUDA=1", f'-DVELOMIND_PROJECT_ROOT="{ref}"']
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    cpp, cu = sources(ref)
    jobs = []
    for s in cpp:
        o = os.path.join(obj, s[len(ref):].strip("/").replace("/", "_") + ".o")
        jobs.append((o, ["g++", "-std=c++23", "-O2", "-mavx2", "-mfma", "-include", "limits", *inc, *defs,
                         f"-I{cuda_home}/include", "-c", s, "-o", o]))
    driver_obj = os.path.join(obj, "reference_driver.o")
    jobs.append((driver_obj, ["g++", "-std=c++23", "-O2", "-include", "limits", *inc, *defs, "-c",
                              os.path.join(HERE, "reference_driver.cpp"), "-o", driver_obj]))
    for s in cu:
        o = os.path.join(obj, s[len(ref):].strip("/").replace("/", "_") + ".o")
        jobs.append((o, [nvcc, "-std=c++20", "-O2", "-gencode", "arch=compute_100,code=sm_100", *inc, *defs,
                         "-c", s, "-o", o]))

    def run(job):
        o, cmd = job
        if os.path.isfile(o) and not force:
            return o
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compiling {cmd[-3]} failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}")
        return o

    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 4)) as pool:
        objs = list(pool.map(run, jobs))
    libs = [f"-L{cuda_home}/lib64", "-lcublas", "-lcudart", "-lpthread", f"-Wl,-rpath,{cuda_home}/lib64"]
    bench_objs = [o for o in objs if o != driver_obj]
    driver_objs = [o for o in objs if "benchmarks_" not in os.path.basename(o)]
    for exe, group in ((EXE, bench_objs), (DRIVER, driver_objs)):
        r = subprocess.run(["g++", "-o", exe, *group, *libs], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {os.path.basename(exe)} failed:\n{r.stderr[-4000:]}")
    return EXE


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE, force="--force" in sys.argv))
