"""Builds libtflite_b200_delegate.so (the TfLiteDelegate plugin) in-tree.

The delegate is compiled against the LiteRT C headers where they lie in a LiteRT checkout
(environment variable LITERT_ROOT); two of its small C sources (TfLiteIntArray helpers) are
compiled from there too. Without the checkout an already built library is kept as is.

The checkout is found through LITERT_ROOT or, when that is unset, as a directory named
`reference` beside this repository.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc", "delegate")
LIB = os.path.join(HERE, "lib")


def litert_root():
    """The LiteRT checkout: $LITERT_ROOT, else a sibling directory `reference` of this repository
    (whether it exists is the caller's question)."""
    env = os.environ.get("LITERT_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


LITERT_ROOT = litert_root()
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
OUT = os.path.join(LIB, "libtflite_b200_delegate.so")
# the LiteRT accelerator definition, under the file name the LiteRT environment loads
ACCELERATOR = os.path.join(LIB, "libLiteRtGpuAccelerator.so")
GEN = os.path.join(LIB, "gen")


def generated_include_dir():
    """litert/build_common/build_config.h is a generated header in the reference build (from
    build_config.h.in, two 0/1 switches): produce it the same way, with GPU and NPU enabled."""
    src = os.path.join(LITERT_ROOT, "litert", "build_common", "build_config.h.in")
    dst = os.path.join(GEN, "litert", "build_common", "build_config.h")
    if os.path.exists(src) and (not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src)):
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        text = open(src).read()
        for name in ("LITERT_BUILD_CONFIG_DISABLE_GPU", "LITERT_BUILD_CONFIG_DISABLE_NPU"):
            text = text.replace(f"#cmakedefine01 {name}", f"#define {name} 0")
        with open(dst, "w") as out:
            out.write(text)
    return GEN


def build_accelerator(force=False):
    """libLiteRtGpuAccelerator.so exporting LiteRtAcceleratorImpl; needs the LiteRT headers."""
    header = os.path.join(LITERT_ROOT, "litert", "c", "internal", "litert_accelerator_def.h")
    if not os.path.exists(header):
        return ACCELERATOR if os.path.exists(ACCELERATOR) else None
    delegate = build(force)
    src = os.path.join(CSRC, "litert_accelerator.cc")
    if not force and not _newer(ACCELERATOR, [src, delegate]):
        return ACCELERATOR
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-shared", "-o", ACCELERATOR, src,
                           "-I" + generated_include_dir(), "-I" + LITERT_ROOT, "-L" + LIB, "-ltflite_b200_delegate",
                           "-Wl,-rpath,$ORIGIN"])
    return ACCELERATOR


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False):
    have_headers = os.path.exists(os.path.join(LITERT_ROOT, "tflite", "core", "c", "common.h"))
    if not have_headers:
        return OUT if os.path.exists(OUT) else None
    from . import build as kernels_build

    kernels = kernels_build.build_kernels(force)
    srcs = [os.path.join(CSRC, f) for f in ("b200_delegate.cc", "device_arena.cc")]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [kernels]
    deps += [os.path.join(os.path.dirname(HERE), "include", f) for f in ("litert_b200.h", "litert_b200_delegate.h")]
    if not force and not _newer(OUT, deps):
        return OUT
    ref_srcs = [os.path.join(LITERT_ROOT, "tflite", "core", "c", "common.cc"),
                os.path.join(LITERT_ROOT, "tflite", "array.cc")]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-shared", "-o", OUT] + srcs + ref_srcs + [
        "-I" + LITERT_ROOT, "-I" + os.path.join(CUDA_HOME, "include"),
        "-L" + LIB, "-llitert_b200", "-Wl,-rpath,$ORIGIN",
        "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    subprocess.check_call(cmd)
    return OUT
