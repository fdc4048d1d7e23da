"""Builds libspinf_b200.so (the C-ABI library of sm_100a kernels) in place with nvcc.

    python -m spinf_serve_b200.csrc.build [--force] [--verbose]

Every translation unit is compiled for sm_100a only (-gencode arch=compute_100a,code=sm_100a); objects are cached next to the
sources and rebuilt when a source or header is newer."""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libspinf_b200.so")
SOURCES = ["host_util.cpp", "abi.cpp", "tile_desc.cpp", "gemm.cu", "glue.cu", "attn_tree.cu", "w4_gemm.cu", "gdn.cu", "gdn_chunk.cu", "gdn_tree.cu", "gdn_tree_tc.cu", "x_attn.cu", "w4_small.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-Wall",
    "-Xptxas",
    "-v",
]


def _headers():
    hs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "..", "include", "spinf_b200.h"))
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _compile(src, force, verbose):
    path = os.path.join(HERE, src)
    obj = os.path.join(HERE, "build", src + ".o")
    if not (force or _stale(obj, [path, __file__] + _headers())):
        return obj, ""
    cmd = [NVCC, *FLAGS, "-x", "cu", "-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, (r.stderr if verbose else "")


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(HERE, s))]
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    objs = [o for o, _ in results]
    for _, log in results:
        if log:
            sys.stderr.write(log)
    if force or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build("--force" in sys.argv, "--verbose" in sys.argv))
