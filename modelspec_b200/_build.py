"""Builds the CUDA backend (libmsx.so) in the package directory with nvcc, for sm_100a only."""
import concurrent.futures
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libmsx.so")

SOURCES = ["cuda/pointwise.cu", "cuda/reduce.cu", "cuda/rowwise.cu", "cuda/embedding.cu", "cuda/gemm.cu", "cuda/gemm_tc.cu", "cuda/gemm_bf16.cu",
           "cuda/attention.cu", "cuda/attention_tc.cu", "cuda/attention_fused.cu", "cuda/optimizer.cu", "cuda/heldout.cu", "cuda/runtime.cu", "cuda/noalloc.cu", "cuda/peer_reduce.cu", "host/training.cpp", "host/packed.cpp", "host/dense.cpp", "host/checkpoint.cpp"]

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-fmad=false", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function"]
# Extra defines for tuning builds, e.g. MSX_NVCC_DEFINES="-DMSX_TC_TRACE".
NVCC_FLAGS += os.environ.get("MSX_NVCC_DEFINES", "").split()


def _obj(src):
    return os.path.join(OBJ, os.path.basename(src).rsplit(".", 1)[0] + ".o")


def _headers():
    out = []
    for root in (os.path.join(CSRC, "cuda"), os.path.join(CSRC, "core"), os.path.join(os.path.dirname(HERE), "include")):
        for name in os.listdir(root):
            if name.endswith((".hpp", ".cuh", ".h")):
                out.append(os.path.join(root, name))
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compiles every .cu of the backend and links libmsx.so; returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    jobs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = _obj(src)
        if force or _stale(obj, [path] + headers):
            jobs.append((path, obj))

    def compile_one(job):
        path, obj = job
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (path, r.stderr))
        return r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        logs = list(pool.map(compile_one, jobs))
    objs = [_obj(s) for s in SOURCES]
    if jobs or force or _stale(LIB, objs):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s" % r.stderr)
    if verbose:
        print("\n".join(logs))
    return LIB


if __name__ == "__main__":
    print(build_library(verbose=True))
