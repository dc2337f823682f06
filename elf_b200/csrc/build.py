"""Build the native extension in-tree: ``python -m elf_b200.csrc.build``.

nvcc cross-compiles for sm_100a without a GPU; the resulting shared object stays next to
the sources (``elf_b200/csrc/_build``) so it ships with the tree to GPU machines.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD_DIR = HERE / "_build"
NAME = "elf_b200_C"
SOURCES = ["bindings.cpp", "fused_bindings.cpp", "host_runtime.cpp", "symm_runtime.cpp", "gemm_sm100.cu", "gemm_sm100_2cta.cu", "fused_ops.cu"]
OPTIONAL_SOURCES = ["attention_sm100.cu", "attention_bwd_sm100.cu", "attention_bindings.cpp", "dp_reduce.cu", "p2p_signal.cu", "dp_reduce_bindings.cpp"]
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "--use_fast_math",
]


NOALLOC_LIB = "libelfb_noalloc.so"


def build_noalloc_library(verbose: bool = False) -> Path:
    """Stand-alone shared library (no PyTorch dependency) with the allocation-free entry point
    of ``rmsnorm_bwd_noalloc.h``; callers load it with ``dlopen`` / ``ctypes``."""
    import subprocess

    BUILD_DIR.mkdir(exist_ok=True)
    out = BUILD_DIR / NOALLOC_LIB
    srcs = [HERE / "rmsnorm_bwd_noalloc.cu", HERE / "fused_ops.cu"]
    deps = srcs + [HERE / "rmsnorm_bwd_noalloc.h", HERE / "fused_ops.h"]
    if out.exists() and all(out.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return out
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC", *NVCC_FLAGS, "-cudart", "shared", "-o", str(out), *map(str, srcs)]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return out


def sources():
    out = [str(HERE / s) for s in SOURCES]
    out += [str(HERE / s) for s in OPTIONAL_SOURCES if (HERE / s).exists()]
    return out


CHECK_NAME = "elf_b200_C_check"
CHECK_BUILD_DIR = HERE / "_build_check"


def build(verbose: bool = False, bounds_check: bool = False):
    """Compile (incrementally, through ninja) and import the extension module.  With
    ``bounds_check`` the debug variant is built instead (``-DELF_BOUNDS_CHECK``: tiled TMA copies
    validate their coordinates on the device, record a violation in the status word and skip the
    copy); it lives beside the regular build under another name and ``ELF_B200_BOUNDS_CHECK=1``
    makes ``elf_b200.ops._ext`` load it."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 1)))
    from torch.utils import cpp_extension

    build_dir = CHECK_BUILD_DIR if bounds_check else BUILD_DIR
    build_dir.mkdir(exist_ok=True)
    defines = ["-DELF_BOUNDS_CHECK"] if bounds_check else []
    if (HERE / "attention_sm100.cu").exists():
        defines.append("-DELFB_WITH_ATTENTION")
    if (HERE / "dp_reduce.cu").exists():
        defines.append("-DELFB_WITH_DP_REDUCE")
    if not bounds_check:
        build_noalloc_library(verbose)
    return cpp_extension.load(
        name=CHECK_NAME if bounds_check else NAME,
        sources=sources(),
        extra_cflags=["-O3", "-std=c++17"] + defines,
        extra_cuda_cflags=NVCC_FLAGS + defines,
        extra_ldflags=["-lcudart"],
        build_directory=str(build_dir),
        with_cuda=True,
        verbose=verbose,
    )


if __name__ == "__main__":
    mod = build(verbose="-v" in sys.argv, bounds_check="--bounds-check" in sys.argv)
    print("built", mod.__file__)
