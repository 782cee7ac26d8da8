r"""
In-tree build of the native extension for sm_100a.

``python -m fastmoe_b200.build`` compiles ``csrc/`` with
``-gencode arch=compute_100a,code=sm_100a`` (the only target; the reference's ``setup.py``
passes no architecture flag at all and leaves the choice to ``TORCH_CUDA_ARCH_LIST``) and
leaves ``fastmoe_b200/_build/fmoe_b200_native.so``.  nvcc cross-compiles, so no GPU is needed
to build.  Environment: ``MOE_DEBUG=1`` adds ``-DMOE_DEBUG`` (as in the reference's
``setup.py:32-33``), ``FMOE_BUILD_VERBOSE=1`` shows the compiler commands.
"""
import glob
import os
import sys

from .ops import native

CSRC = os.path.join(native.PKG_DIR, "csrc")

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
]


def sources():
    files = []
    for pattern in ("*.cpp", "cpu/*.cpp", "runtime/*.cpp", "sm100/*.cpp", "sm100/*.cu"):
        files.extend(sorted(glob.glob(os.path.join(CSRC, pattern))))
    return files


def _newest_source_mtime():
    newest = 0.0
    for root, _dirs, names in os.walk(CSRC):
        for name in names:
            newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def is_fresh():
    so = native.so_path()
    return os.path.exists(so) and os.path.getmtime(so) >= _newest_source_mtime()


def build(force=False, verbose=None):
    r"""Compile (when stale) and return the path of the shared object."""
    if not force and is_fresh():
        return native.so_path()
    from torch.utils import cpp_extension
    os.makedirs(native.BUILD_DIR, exist_ok=True)
    if verbose is None:
        verbose = os.environ.get("FMOE_BUILD_VERBOSE", "0") == "1"
    cflags = ["-O3", "-std=c++17"]
    cuda_flags = list(CUDA_FLAGS)
    if os.environ.get("MOE_DEBUG", "0") == "1":
        cflags.append("-DMOE_DEBUG")
        cuda_flags.append("-DMOE_DEBUG")
    os.environ.setdefault("MAX_JOBS", "8")
    cpp_extension.load(
        name=native.MODULE_NAME,
        sources=sources(),
        extra_cflags=cflags,
        extra_cuda_cflags=cuda_flags,
        extra_include_paths=[CSRC],
        build_directory=native.BUILD_DIR,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    return native.so_path()


if __name__ == "__main__":
    path = build(force="--force" in sys.argv)
    print(path)
