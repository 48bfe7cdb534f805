"""Builds libb2q.so (hand-written CUDA for sm_100a + the C ABI) in-tree with nvcc.

    python llm-scaler_b200/build.py [--force] [--verbose]

Every csrc/*.cu is compiled to build/*.o in parallel (only when the source or a
header is newer than the object) and linked into
custom_esimd_kernels_vllm/libb2q.so.  nvcc cross-compiles without a GPU.
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
OUT = os.path.join(HERE, "custom_esimd_kernels_vllm", "libb2q.so")
OUT_TORCH = os.path.join(HERE, "custom_esimd_kernels_vllm", "libb2q_torch.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I", INCLUDE,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libb2q.so cannot be built")


def _newest_header():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "b2q.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(nvcc, src, obj, verbose):
    extra = os.environ.get("B2Q_EXTRA_NVCC_FLAGS", "").split()      # e.g. -DB2Q_UMMA_PROF for in-kernel wait timers
    cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return r.stderr if verbose else ""


def build(force=False, verbose=False):
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_time = _newest_header()
    jobs, objs = [], []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs):
                if log:
                    sys.stderr.write(log)
    if jobs or not os.path.exists(OUT):
        cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    build_torch_ops(force or bool(jobs))
    return OUT


def build_torch_ops(force=False):
    """libb2q_torch.so: the C++ torch-op registration of the dense linears (csrc/torch_ops.cpp) over libb2q.so.
    Host code only: compiled with g++ against the installed torch's headers and linked with its libraries."""
    src = os.path.join(CSRC, "torch_ops.cpp")
    hdr = os.path.join(INCLUDE, "b2q.h")
    if not force and os.path.exists(OUT_TORCH) and os.path.getmtime(OUT_TORCH) >= max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(OUT)):
        return OUT_TORCH
    import torch
    tdir = os.path.dirname(torch.__file__)
    cuda_home = os.environ.get("CUDA_HOME") or os.path.dirname(os.path.dirname(_nvcc()))
    gxx = os.environ.get("CXX") or shutil.which("g++")
    if not gxx:
        raise RuntimeError("g++ not found; libb2q_torch.so cannot be built")
    cmd = [gxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I", INCLUDE, "-I", os.path.join(tdir, "include"), "-I", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           "-I", os.path.join(cuda_home, "include"), src, "-o", OUT_TORCH,
           "-L", os.path.dirname(OUT), "-l:libb2q.so", "-L", os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
           "-lc10", "-lc10_cuda", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return OUT_TORCH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
