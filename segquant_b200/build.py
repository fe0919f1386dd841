"""Ahead-of-time build of libsegquant_b200.so with nvcc for sm_100a.

The reference JIT-builds five pybind11 modules against CUTLASS through
torch.utils.cpp_extension.load (segquant/utils/extension.py:25-64).  This library has no torch or
CUTLASS dependency: a handful of .cu files plus the C ABI, linked with the static CUDA runtime so the
.so also loads on a machine without a GPU driver (symbol checks, CPU tests).

    python -m segquant_b200.build          # build if sources are newer than the .so
    python -m segquant_b200.build --force
"""
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libsegquant_b200.so")
SOURCES = ["capi.cu", "act_quant.cu", "weight_quant.cu", "seg_gemm.cu", "seg_gemv.cu", "static_scratch.cu", "gated_residual.cu", "peer_push.cu",
           # one translation unit per (kind, DualScale): the GEMM kernels dominate compile time and build in parallel
           "seg_gemm_tu_i8.cu", "seg_gemm_tu_i8_dual.cu", "seg_gemm_tu_f8.cu", "seg_gemm_tu_f8_dual.cu",
           "seg_gemm_tu_w4.cu", "seg_gemm_tu_w4_dual.cu"]
HEADERS = [os.path.join(CSRC, h) for h in ("common.cuh", "seg_gemm_params.cuh", "seg_gemm_kernels.cuh", "seg_gemm_2cta.cuh",
                                           "seg_gemm_epilogue.cuh")] + [os.path.join(PKG_DIR, "..", "include", "segquant_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-cudart", "static",
]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, ptxas_verbose=False, extra_flags=(), out=None):
    """Compile every CUDA source for sm_100a and link the shared library in-tree.

    extra_flags / out: build a variant (e.g. ["-DSQ_TRACE"]) into another file without touching the
    product library."""
    variant = out is not None
    target = out or LIB_PATH
    if not variant and not force and not needs_build():
        return LIB_PATH
    objs = []
    procs = []
    for s in SOURCES:
        obj = os.path.join(CSRC, s.replace(".cu", ".variant.o" if variant else ".o"))
        cmd = [_nvcc()] + NVCC_FLAGS + list(extra_flags) + (["-Xptxas", "-v"] if ptxas_verbose else []) + [
            "-c", os.path.join(CSRC, s), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"[segquant_b200.build] nvcc failed on {s}:\n{out}\n")
        elif verbose or ptxas_verbose:
            print(out)
    if failed:
        raise RuntimeError("segquant_b200: CUDA compilation failed")
    link = [_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
            "-o", target] + objs
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("segquant_b200: link failed:\n" + r.stdout)
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_verbose="--ptxas" in sys.argv)
    print(path)
