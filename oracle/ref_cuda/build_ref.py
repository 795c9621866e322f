"""Builds oracle/_ref/libenergon_ref.so: the reference's own CUDA kernels, recompiled for
sm_100a from the reference checkout where it lies, behind the C shim next to this file.

    python oracle/ref_cuda/build_ref.py [--force]

TEST INFRASTRUCTURE (see oracle/__init__.py).  The reference's setup.py (lines 119-147) builds
the same sources with `-O3 --use_fast_math -std=c++14` for sm_70 / sm_80 only; here the flags
are kept except for the standard (c++17, which torch's headers need today) and the
architecture.  Nothing is copied: the three .cu files are compiled in place and only objects
and the library are written, under oracle/_ref/ (git-ignored).  Where no checkout exists (the
GPU box) the prebuilt library that travelled with the repository is used as it is.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(ROOT, "oracle", "_ref")
LIB = os.path.join(OUT, "libenergon_ref.so")
SOURCES = ("scale_mask_softmax_kernel.cu", "transpose_pad_fusion_kernel.cu", "layer_norm_cuda_kernel.cu")


def reference_csrc():
    root = os.environ.get("ENERGONAI_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
    path = os.path.join(root, "energonai", "kernel", "cuda_native", "csrc")
    return path if os.path.isdir(path) else None


def build(force=False):
    """Returns the library path, or None when neither the checkout nor a prebuilt library exists."""
    csrc = reference_csrc()
    if csrc is None:
        return LIB if os.path.exists(LIB) else None
    shim = os.path.join(HERE, "ref_shim.cu")
    inputs = [os.path.join(csrc, s) for s in SOURCES] + [shim]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(p) <= os.path.getmtime(LIB) for p in inputs):
        return LIB
    from torch.utils.cpp_extension import include_paths, library_paths
    os.makedirs(OUT, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-std=c++17",
             "-DVERSION_GE_1_1", "-DVERSION_GE_1_3", "-DVERSION_GE_1_5",
             "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
             "-DTHRUST_IGNORE_CUB_VERSION_CHECK", "-Xcompiler", "-fPIC", "-w", "-I", csrc]
    for inc in include_paths("cuda") if "device_type" in include_paths.__code__.co_varnames else include_paths():
        flags += ["-isystem", inc]
    objs, procs = [], []
    for src in inputs:
        obj = os.path.join(OUT, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen([nvcc] + flags + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed for {src}")
    libdirs = library_paths("cuda") if "device_type" in library_paths.__code__.co_varnames else library_paths()
    link = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    for d in libdirs:
        link += ["-L", d, "-Xlinker", "-rpath", "-Xlinker", d]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link of libenergon_ref.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
