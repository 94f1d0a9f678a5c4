"""Build libbiloco_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m biloco_b200.csrc.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libbiloco_b200.so")
SOURCES = ["api.cu", "lowrank_ref.cu", "act_quant.cu", "decode_attn.cu", "fp4_gemm_simt.cu", "peel.cu", "peer_reduce.cu", "fused_linear.cu"]
HEADERS = ["ptx.cuh", "schedule.h", "fused_cfg.cuh", "fused_lowrank.cuh", "fused_kernel.cuh", "ztc_kernel.cuh", "slab_kernel.cuh", "slab_plain_kernel.cuh", "slab_host.cuh", "quant_math.cuh", os.path.join("..", "..", "include", "biloco_b200.h")]


def _nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), "-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-O3",
           "-o", LIB] + [os.path.join(HERE, s) for s in SOURCES] + ["-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libbiloco_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
