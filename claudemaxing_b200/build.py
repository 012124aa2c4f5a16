"""Builds libsoup_b200.so from claudemaxing_b200/csrc with nvcc for sm_100a, in tree.

The shared library is the only native artefact of the package. It is compiled next to its sources
(`claudemaxing_b200/csrc/libsoup_b200.so`) so that a checkout that was built once can be copied to
a GPU machine as it is. `python -m claudemaxing_b200.build` rebuilds it; `build(force=False)`
rebuilds only when a source is newer than the library.
"""

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libsoup_b200.so")
OBJ_DIR = os.path.join(CSRC, "build")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--use_fast_math",
              "-Xptxas", "-v"]
# --use_fast_math only affects the transcendental intrinsics the elementwise kernels opt into; every
# product that must be bit-exact is written with __fmul_rn/__fadd_rn, which it does not touch.


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: libsoup_b200.so cannot be built")
    return path


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "soup_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def _compile_one(nvcc, src, log):
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log.append((src, proc.stdout + proc.stderr))
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
    return obj


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ for sm_100a and link libsoup_b200.so. Returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    log = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(nvcc, s, log), sources()))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", LIB, *objs, "-lcudart_static", "-ldl", "-lrt",
            "-lpthread"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    with open(os.path.join(OBJ_DIR, "ptxas.log"), "w") as f:
        for src, text in log:
            f.write(f"==== {src}\n{text}\n")
    if verbose:
        for src, text in log:
            print(f"==== {src}\n{text}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv or True, verbose="-v" in sys.argv))
