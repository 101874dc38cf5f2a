"""Builds the sm_100a extension in-tree: ``chatlearn_b200/_C.so``.

nvcc cross-compiles for ``compute_100a / sm_100a`` (no GPU needed); the shared
object sits next to the Python package so it ships with a source snapshot.
Run ``python -m chatlearn_b200.csrc.build`` or call ``build()``.
"""
import fcntl
import glob
import hashlib
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


_MARK = b"CLB200_SRC_HASH="


def source_hash() -> str:
    """Hash of everything the binary is made from: the CUDA/C++ sources, their headers and this
    file (the compiler flags live here).  It is baked into the shared object, so a binary that
    does not match the sources beside it is detected before any kernel is looked up."""
    h = hashlib.sha256()
    deps = sources() + sorted(glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h"))) \
        + [os.path.abspath(__file__)]
    for path in deps:
        h.update(os.path.basename(path).encode() + b"\0")
        h.update(open(path, "rb").read())
    return h.hexdigest()[:32]


def binary_hash(path: str = TARGET):
    """The source hash baked into a built shared object (None: no binary, or one built without it)."""
    try:
        blob = open(path, "rb").read()
    except OSError:
        return None
    i = blob.find(_MARK)
    return blob[i + len(_MARK):i + len(_MARK) + 32].decode("ascii", "replace") if i >= 0 else None


def is_stale() -> bool:
    return binary_hash() != source_hash()


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not is_stale():
        return TARGET
    os.makedirs(os.path.join(PKG, "build"), exist_ok=True)
    # one builder at a time: the ranks of a job that all find a stale binary queue up here and all
    # but the first find it fresh
    with open(os.path.join(PKG, "build", ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not is_stale():
            return TARGET
        return _build_locked(verbose)


def _build_locked(verbose: bool) -> str:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")   # placeholder; real arch comes from NVCC_FLAGS
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils import cpp_extension
    build_dir = os.path.join(PKG, "build", "ext")
    os.makedirs(build_dir, exist_ok=True)
    stamp = os.path.join(build_dir, "src_hash.cpp")
    text = ('extern "C" const char clb200_src_hash[] = "%s%s";\n'
            'const char* clb200_source_hash() { return clb200_src_hash + %d; }\n'
            % (_MARK.decode(), source_hash(), len(_MARK)))
    if not os.path.exists(stamp) or open(stamp).read() != text:
        open(stamp, "w").write(text)
    cpp_extension.load(name="_C", sources=sources() + [stamp], extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=NVCC_FLAGS, extra_ldflags=["-lcuda"] if False else [],
                       build_directory=build_dir, verbose=verbose, is_python_module=False)
    built = os.path.join(build_dir, "_C.so")
    shutil.copyfile(built, TARGET + ".tmp")
    os.replace(TARGET + ".tmp", TARGET)
    return TARGET


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
