"""Builds libmldfc.so (the CUDA kernels and their C ABI) in-tree with nvcc for
sm_100a.  Usage: python build.py [--force] [--verbose] [--trace]
--trace compiles the kernels' tuning instrumentation (per-CTA timestamps and the
mld_debug_* entry points that read them) into the library; the default build has
neither."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libmldfc.so")

SOURCES = ["api.cu", "pack_kernels.cu", "gemv_generic.cu", "gemv_stream.cu", "decode_step.cu", "decode_mega.cu",
           "gemm_umma.cu", "gemm_pair.cu", "gemm_wtmem.cu", "shard_group.cu", "embedding.cu", "loader.cu"]
HEADERS = ["common.cuh", "kernels.h", "nccl_lazy.h", "pair_common.cuh", os.path.join(ROOT, "include", "mldfc.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False, trace=False):
    """Compiles every CUDA source of the package into one shared library."""
    if not force and not trace and not _stale():
        return OUT
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for s in SOURCES:
        obj = os.path.join(HERE, "build", s.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, s), "-o", obj]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        if trace:
            cmd += ["-DMLD_TRACE"]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if out.strip():
            print(f"--- {s}\n{out}")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [_nvcc(), "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    cmd += ["-ldl"]
    subprocess.check_call(cmd)
    return OUT


HOST_TEST = os.path.join(HERE, "build", "host_test")


def build_host_test(force=False):
    """Compiles the C++ host mirror and its test program against libmldfc.so (g++ only)."""
    build()
    srcs = [os.path.join(HERE, "host", "tests", "host_test.cc"), os.path.join(HERE, "host", "mld_host.cc")]
    deps = srcs + [os.path.join(HERE, "host", "mld_host.h"), OUT]
    if not force and os.path.exists(HOST_TEST) and all(os.path.getmtime(d) <= os.path.getmtime(HOST_TEST) for d in deps):
        return HOST_TEST
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-O2", "-std=c++17", "-Wall", "-o", HOST_TEST, *srcs, "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(cuda, "include"), "-L", HERE, "-lmldfc", "-L", os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath," + HERE, "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    subprocess.check_call(cmd)
    return HOST_TEST


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
