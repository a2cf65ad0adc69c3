"""Builds the native libraries of the package in-tree with nvcc for sm_100a.

    python -m litert_b200.build            # kernels + C ABI (+ delegate when the LiteRT headers are found)

Outputs go to litert_b200/lib/. Cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden"]
COMMON += os.environ.get("B200_NVCC_FLAGS", "").split()  # e.g. -DB200_UMMA_KB=108 (shared-memory budget of a GEMV CTA)

KERNEL_SOURCES = ["pack.cu", "fc_umma.cu", "fc_w4_umma.cu", "fc_w4_gemv.cu", "sdpa_decode.cu", "decoder_kernels.cu", "decoder.cu", "shim.cu", "sdpa_static.cu", "glue_abi.cu", "peak_probe.cu", "elementwise.cu"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _all_deps():
    deps = []
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for dirpath, _, files in os.walk(root):
            deps += [os.path.join(dirpath, f) for f in files]
    return deps


def build_kernels(force=False, verbose=False):
    os.makedirs(LIB, exist_ok=True)
    out = os.path.join(LIB, "liblitert_b200.so")
    srcs = [os.path.join(CSRC, s) for s in KERNEL_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if not force and not _newer(out, _all_deps()):
        return out
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(LIB, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
        procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    cmd = [NVCC] + ARCH + ["-shared", "-o", out] + objs
    subprocess.check_call(cmd)
    for o in objs:
        os.remove(o)
    return out


def build_all(force=False, verbose=False):
    paths = [build_kernels(force, verbose)]
    try:
        from . import build_delegate
    except ImportError:
        build_delegate = None
    if build_delegate is not None:
        p = build_delegate.build(force)
        if p:
            paths.append(p)
        a = build_delegate.build_accelerator(force)
        if a:
            paths.append(a)
    return paths


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print(p)
