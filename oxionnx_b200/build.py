"""Builds oxionnx_b200/_lib/liboxb200.so: the CUDA kernels (sm_100a only) plus the C++ host
runtime behind the C ABI of include/oxb200.h.

nvcc cross-compiles without a GPU.  The CUDA runtime is linked statically and the driver's
tensor-map encoders are resolved at run time, so the library loads (and its symbols can be
checked) on a host that has no GPU driver.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "liboxb200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-ffp-contract=off,-fno-fast-math", "--fmad=false"]
# --fmad=false everywhere except the tensor-core kernel file, whose float epilogue is one add
SOURCES = {
    "kernels_glue.cu": COMMON,
    "kernels_simt.cu": [f for f in COMMON if f != "--fmad=false"],
    "kernels_umma.cu": [f for f in COMMON if f != "--fmad=false"],
    "umma_i8.cu": [f for f in COMMON if f != "--fmad=false"],
    "umma_tf32.cu": [f for f in COMMON if f != "--fmad=false"],
    "umma_f16.cu": [f for f in COMMON if f != "--fmad=false"],
    "umma_probe.cu": [f for f in COMMON if f != "--fmad=false"],
    "umma_chain.cu": [f for f in COMMON if f != "--fmad=false"],
    "umma_attention.cu": [f for f in COMMON if f != "--fmad=false"],
    "runtime.cpp": COMMON,
    "planner.cpp": COMMON,
    "abi.cpp": COMMON,
    "onnx_model.cpp": COMMON,
    "model_abi.cpp": COMMON,
}
HEADERS = ["common.hpp", "kernels.hpp", "runtime.hpp", "umma_kernel.cuh", "umma_launch.cuh", "umma_chain.cuh", "model.hpp", "abi_internal.hpp", os.path.join("..", "..", "include", "oxb200.h")]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src, flags in SOURCES.items():
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc] + ARCH + flags + ["-x", "cu", "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for log in ex.map(run, jobs):
                if verbose and log:
                    print(log)
    if force or jobs or _stale(LIB, objs):
        run([nvcc] + ARCH + ["-shared", "-o", LIB] + objs + ["-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
