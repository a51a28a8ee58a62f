"""Builds the sm_100a shared library and the Driver-API cubin in-tree with nvcc (no JIT cache, no torch extension).

    python -m turkce_llm_b200.build [--force] [--verbose]

Outputs: turkce_llm_b200/libturkce_b200.so (the C ABI of include/turkce_b200.h) and
turkce_llm_b200/turkce_b200_gemm.cubin (the GEMM family under the reference's kernel names, for the reference's
cuModuleLoadData loader).  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libturkce_b200.so")
CUBIN = os.path.join(HERE, "turkce_b200_gemm.cubin")
CUBIN_SRC = os.path.join(CSRC, "cubin", "gemm_ref_abi.cu")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if os.path.isfile(os.path.join(CSRC, f))] + \
           [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return any(os.path.getmtime(d) > t for d in deps)


def build_cubin(force=False, verbose=False):
    """nvcc -cubin of the reference-ABI GEMM kernels (a module image for cuModuleLoadData)."""
    deps = [CUBIN_SRC, os.path.join(CSRC, "ptx.cuh")]
    if not force and os.path.exists(CUBIN) and all(os.path.getmtime(d) <= os.path.getmtime(CUBIN) for d in deps):
        return CUBIN
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17"] + \
          (["-Xptxas", "-v"] if verbose else []) + ["-o", CUBIN, CUBIN_SRC]
    subprocess.check_call(cmd)
    return CUBIN


def build(force=False, verbose=False):
    build_cubin(force, verbose)
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + os.environ.get("TB_NVCC_FLAGS", "").split() + (["-Xptxas", "-v"] if verbose else []) + ["-I", INCLUDE, "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (os.path.basename(src), out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
