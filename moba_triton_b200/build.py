"""Builds libmoba_b200.so in-tree with nvcc for sm_100a.

    python -m moba_triton_b200.build [--force] [--verbose]

Every csrc/*.cu is compiled to an object (in parallel) and linked into
`moba_triton_b200/libmoba_b200.so`. The library links the static CUDA runtime
only; the driver entry points it needs (tensor-map encoding) are resolved at
run time, so it loads on machines without a GPU driver.
"""

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libmoba_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest_dep() -> float:
    deps = glob.glob(os.path.join(CSRC, "*.cu*")) + glob.glob(os.path.join(PKG, "..", "include", "*.h"))
    return max(os.path.getmtime(p) for p in deps)


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles what is out of date and returns the library path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    newest_header = max([os.path.getmtime(p) for p in glob.glob(os.path.join(CSRC, "*.cuh"))
                         + glob.glob(os.path.join(PKG, "..", "include", "*.h"))] or [0.0])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj)
                and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_header)):
            return obj
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    # drop objects whose source no longer exists
    keep = set(objs)
    for stale in glob.glob(os.path.join(OBJ, "*.o")):
        if stale not in keep:
            os.remove(stale)
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link of libmoba_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
