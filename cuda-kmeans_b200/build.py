"""Builds libbkm.so (the C-ABI library, include/bkm.h) in-tree with nvcc for sm_100a.

    python cuda-kmeans_b200/build.py [--force] [--verbose]

The library links the CUDA runtime statically and resolves NCCL and the driver's tensor-map
encoder at run time, so it loads on a machine without a GPU (where every compute entry point
then fails with BKM_ERR_CUDA).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbkm.so")
SOURCES = ["api.cu", "assign_simt.cu", "assign_tc.cu", "assign_tc_pair.cu", "update.cu", "no_alloc.cu", "f64.cu"]
HEADERS = ["common.cuh", "kernels.cuh", "ptx.cuh", "tc_common.cuh", "keys.cuh", os.path.join("..", "..", "include", "bkm.h")]
CLI_SRC = os.path.join(HERE, "cli", "bkm_kmeans.cpp")
CLI = os.path.join(HERE, "bkm-kmeans")
CLI2_SRC = os.path.join(HERE, "cli", "bkm_bucketing.cpp")
CLI2 = os.path.join(HERE, "bkm-bucketing")
CLI_HEADERS = [os.path.join(HERE, "cli", "reference_data.hpp")]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = _sources() + [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compiles every .cu of the library into one shared object; returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in _sources():
        obj = src[:-3] + ".o"
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + out + "\n")
        failed = failed or p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-ldl"]
    subprocess.check_call(link)
    return LIB


def build_cli(force=False):
    """Compiles the two command-line harnesses (cli/bkm_kmeans.cpp, cli/bkm_bucketing.cpp) next to the
    library; returns the path of the k-means one."""
    lib = build()
    nvcc = os.environ.get("NVCC", "nvcc")
    for src, exe in ((CLI_SRC, CLI), (CLI2_SRC, CLI2)):
        newest = max([os.path.getmtime(src), os.path.getmtime(lib)] + [os.path.getmtime(h) for h in CLI_HEADERS])
        if not force and os.path.exists(exe) and os.path.getmtime(exe) >= newest:
            continue
        cmd = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(HERE, "..", "include"), src,
               "-L", HERE, "-lbkm", "-Xlinker", "-rpath=$ORIGIN", "-o", exe]
        subprocess.check_call(cmd)
    return CLI


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_cli(force="--force" in sys.argv))
