"""Builds the sm_100a cubins, libqmatmul.so and the kernel descriptions.

Usage: python lib_b200/build.py [--force]
nvcc cross-compiles for sm_100a, so this runs on a machine without a GPU.
Outputs (all git-ignored, all next to the sources they come from):
  lib_b200/csrc/build/<name>.sm_100a.cubin   one per .cu file
  lib_b200/csrc/build/<name>.sm_100a.json    kernel table in the field names of the
                                             reference's cudakernel.Artifact
                                             (nvidia/x/cudakernel/artifact.go:104-116)
  lib_b200/libqmatmul.so                     host library with the cubins embedded
"""
import json
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libqmatmul.so")
KERNEL_SOURCES = ["qm_gemv.cu", "qm_dequant.cu", "qm_gemv_q4k.cu", "qm_gemm_q4k.cu", "qm_moe.cu", "qm_gemv_kq.cu", "qm_q8_1.cu"]
HOST_SOURCES = ["qm_host.cpp", "qm_stack.cpp", "qm_moe.cpp", "qm_expert_cache.cpp", "qm_gguf.cpp", "qm_q8_1.cpp", "qm_expert_pool.cpp"]
RUNTIME_SOURCES = ["qm_noalloc.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# QM_DEBUG_BUILD=1 compiles the timing experiments in (phase time stamps, switches that turn
# pipeline roles off and give wrong results). The shipped build leaves it unset.
DEBUG = ["-DQM_DEBUG"] if os.environ.get("QM_DEBUG_BUILD") else []


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


def _describe(src, cubin, ptxas_log):
    """Kernel table for Go callers that load the cubin through nvidia/driver."""
    text = open(src).read()
    names = re.findall(r'QM_(?:GEMV|DD|KQ|DD_SEL|LEAN|DD8)_KERNEL\((\w+),', text) + re.findall(
        r'extern "C" __global__ void\s+(?:__launch_bounds__\([^)]*\)\s*)?(\w+)\(', text)
    res = {}
    cur = None
    for line in ptxas_log.splitlines():
        m = re.search(r"Compiling entry function '(\w+)'", line)
        if m:
            cur = m.group(1)
        m = re.search(r"Used (\d+) registers", line)
        if m and cur:
            res[cur] = {"registers": int(m.group(1))}
    return {"kind": "cubin", "target": "sm_100a", "file": os.path.basename(cubin),
            "kernels": [{"entry_point": n,
                         "schema": [{"name": "args", "kind": "struct_by_value",
                                     "defined_in": "lib_b200/csrc/qm_kernel_args.h"}],
                         "resources": res.get(n, {})} for n in names if n != "name"]}


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "qmatmul.h"))
    cubins = []
    for name in KERNEL_SOURCES:
        src = os.path.join(CSRC, name)
        cubin = os.path.join(OUT, name[:-3] + ".sm_100a.cubin")
        cubins.append(cubin)
        if force or _newer(cubin, [src] + headers):
            log = _run([NVCC] + ARCH + DEBUG + ["-cubin", "-O3", "-lineinfo", "-std=c++17", "-Xptxas", "-v",
                                        "-o", cubin, src])
            if verbose:
                print(log)
            with open(cubin[:-6] + ".json", "w") as f:
                json.dump(_describe(src, cubin, log), f, indent=1)
    srcs = [os.path.join(CSRC, s) for s in HOST_SOURCES]
    # translation units that use the CUDA runtime (kernels launched with <<<>>>)
    rt_objs = []
    for name in RUNTIME_SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(OUT, name[:-3] + ".o")
        rt_objs.append(obj)
        if force or _newer(obj, [src, os.path.join(CSRC, "qm_gemv.cu")] + headers):
            _run([NVCC] + ARCH + DEBUG + ["-c", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                                  "-o", obj, src])
    if force or _newer(LIB, srcs + headers + cubins + rt_objs):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-fvisibility=hidden"] + DEBUG + [
              "-DQM_CUBIN_DIR=" + OUT, "-I/usr/local/cuda/include", "-o", LIB] + srcs + rt_objs +
             ["-L/usr/local/cuda/lib64", "-lcudart_static", "-lrt", "-ldl", "-lpthread"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
