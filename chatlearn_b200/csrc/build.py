"""Builds the sm_100a extension in-tree: ``chatlearn_b200/_C.so``.

nvcc cross-compiles for ``compute_100a / sm_100a`` (no GPU needed); the shared
object sits next to the Python package so it ships with a source snapshot.
Run ``python -m chatlearn_b200.csrc.build`` or call ``build()``.
"""
import glob
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
TARGET = os.path.join(PKG, "_C.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-std=c++17", "--expt-relaxed-constexpr", "-Xptxas", "-v",
              "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "*.cu")) + glob.glob(os.path.join(HERE, "*.cpp")))


def is_stale() -> bool:
    if not os.path.exists(TARGET):
        return True
    t = os.path.getmtime(TARGET)
    deps = sources() + glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h")) \
        + [os.path.abspath(__file__)]          # the flags live in this file
    return any(os.path.getmtime(s) > t for s in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not is_stale():
        return TARGET
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")   # placeholder; real arch comes from NVCC_FLAGS
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils import cpp_extension
    build_dir = os.path.join(PKG, "build", "ext")
    os.makedirs(build_dir, exist_ok=True)
    cpp_extension.load(name="_C", sources=sources(), extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=NVCC_FLAGS, extra_ldflags=["-lcuda"] if False else [],
                       build_directory=build_dir, verbose=verbose, is_python_module=False)
    built = os.path.join(build_dir, "_C.so")
    shutil.copyfile(built, TARGET)
    return TARGET


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
