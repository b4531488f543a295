"""Builds the CUDA library in-tree with nvcc for sm_100a (no JIT cache, no torch).

``python -m deepstrix_b200._build`` or ``build()``; the result is
``deepstrix_b200/libdsx_moe.so`` next to this file.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdsx_moe.so")
# one of the library's kernels as a stand-alone code object, for callers that load kernels by name
# (dsx_module_load_data / dsx_module_get_function / dsx_function_launch)
CUBIN_PATH = os.path.join(_HERE, "kernels", "dsx_combine.cubin")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
EXTRA = os.environ.get("DSX_NVCC_EXTRA", "").split()
FLAGS = EXTRA + [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "--expt-relaxed-constexpr",
]


def sources():
    return sorted(glob.glob(os.path.join(_HERE, "csrc", "*.cu")))


def stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(CUBIN_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(_HERE, "csrc", "*.cuh")) + glob.glob(os.path.join(_HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(p) > t for p in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    if not force and not stale():
        return LIB_PATH
    objs = []
    procs = []
    obj_dir = os.path.join(_HERE, "csrc", "obj")
    os.makedirs(obj_dir, exist_ok=True)
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [NVCC] + [f for f in FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose or ptxas_info:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs
    subprocess.run(cmd, check=True)
    os.makedirs(os.path.dirname(CUBIN_PATH), exist_ok=True)
    subprocess.run([NVCC, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
                    os.path.join(_HERE, "csrc", "combine.cu"), "-o", CUBIN_PATH], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
