"""Build the reference's own CUDA extension for sm_100a, out of tree, as a GPU comparator (test infrastructure).

    python -m oracle.build_ref_kernel [--reference /path/to/BiLoCo] [--jobs 2]

What it does, all outside the repository's tracked files:
  * copies the CUTLASS 4.5 header trees that ship inside the ``flashinfer`` wheel to a temporary directory and applies
    the reference's ``patches/cutlass_biloco.patch`` to that copy (the reference expects a patched CUTLASS checkout as
    a git submodule, which is absent);
  * writes a ten-line ``helper.h`` (the reference includes the CUTLASS examples' helper only for ``CUTLASS_CHECK``);
  * compiles ``csrc/biloco_gemm.cu``, ``csrc/reference_ops.cu`` and ``csrc/bindings.cpp`` where they lie in the reference
    tree (nothing is copied into this repository) with the flags of the reference's ``setup.py`` and
    ``-gencode arch=compute_100a,code=sm_100a``, and links them against the installed torch;
  * leaves exactly one file: ``oracle/_ref/biloco_ref_C.so`` (git-ignored; it travels to the GPU box).

The comparator is loaded only by ``oracle/ref_kernel.py`` in a process of its own (it registers the same
``torch.ops.biloco`` namespace as this package's operators). Needs about 15 minutes and 10 GB of memory.
"""
import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "biloco_ref_C.so")

HELPER_H = """#pragma once
#include <stdexcept>
#include <string>
#include "cutlass/cutlass.h"
#define CUTLASS_CHECK(status)                                                                   \\
    {                                                                                           \\
        cutlass::Status error = status;                                                         \\
        if (error != cutlass::Status::kSuccess)                                                 \\
            throw std::runtime_error(std::string("CUTLASS error: ") + cutlassGetStatusString(error)); \\
    }
"""


def run(cmd, **kw):
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True, **kw)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("BILOCO_REFERENCE", "/root/reference"),
                    help="checkout of the reference (or set BILOCO_REFERENCE)")
    ap.add_argument("--work", default=None, help="scratch directory (default: a fresh temporary one)")
    a = ap.parse_args()
    ref = os.path.abspath(a.reference)
    if not os.path.exists(os.path.join(ref, "csrc", "biloco_gemm.cu")):
        sys.exit(f"reference tree not found at {ref}")
    import flashinfer
    import torch
    from torch.utils import cpp_extension as ce
    cut_src = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
    work = a.work or tempfile.mkdtemp(prefix="biloco_ref_build_")
    os.makedirs(work, exist_ok=True)
    cut = os.path.join(work, "cutlass")
    if not os.path.exists(os.path.join(cut, "include", "cutlass", "gemm", "kernel", "binarysvd_side_hook.hpp")):
        shutil.rmtree(cut, ignore_errors=True)
        os.makedirs(os.path.join(cut, "tools", "util"))
        shutil.copytree(os.path.join(cut_src, "include"), os.path.join(cut, "include"))
        shutil.copytree(os.path.join(cut_src, "tools", "util", "include"), os.path.join(cut, "tools", "util", "include"))
        run(["patch", "-p1", "-d", cut, "-i", os.path.join(ref, "patches", "cutlass_biloco.patch")])
    shim = os.path.join(work, "shim")
    os.makedirs(shim, exist_ok=True)
    with open(os.path.join(shim, "helper.h"), "w") as f:
        f.write(HELPER_H)

    inc = [os.path.join(ref, "csrc"), os.path.join(cut, "include"), os.path.join(cut, "tools", "util", "include"), shim]
    inc += ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    incf = [f"-I{d}" for d in inc]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = ["-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    nvcc = ["nvcc", "-O3", "-std=c++17", "-DNDEBUG", "-gencode=arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
            "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-ffast-math", "-Xcompiler", "-funroll-loops",
            "-Xcompiler", "-finline-functions", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
            "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + defs + incf
    objs = []
    procs = []
    for src in ("biloco_gemm.cu", "reference_ops.cu"):
        o = os.path.join(work, src + ".o")
        objs.append(o)
        cmd = nvcc + ["-c", os.path.join(ref, "csrc", src), "-o", o]
        print("+", " ".join(cmd[:6]), "...", src, flush=True)
        procs.append(subprocess.Popen(cmd))
    o = os.path.join(work, "bindings.o")
    objs.append(o)
    run(["g++", "-O3", "-std=c++17", "-fPIC"] + defs + incf + ["-c", os.path.join(ref, "csrc", "bindings.cpp"), "-o", o])
    for p in procs:
        if p.wait() != 0:
            sys.exit("nvcc failed")
    os.makedirs(OUT_DIR, exist_ok=True)
    libs = [f"-L{d}" for d in ce.library_paths()] + ["-L/usr/local/cuda/lib64"]
    run(["g++", "-shared", "-o", OUT] + objs + libs + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
                                                       "-lcudart", "-lcuda"])
    print(OUT)


if __name__ == "__main__":
    main()
