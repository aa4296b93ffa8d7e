"""In-tree build and loading of the native library.

The CUDA/C++ sources under ``csrc/`` are compiled for sm_100a only into
``flashoverlap_b200/lib/libst_pybinding.so`` (the file name the reference loads,
reference: src/CMakeLists.txt:60-70, example/RowParallelLinear.py:8-9) with
``torch.utils.cpp_extension`` driving ninja.  A digest of the sources is stored
beside the library so that an up-to-date library is loaded directly, without
invoking the compiler.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sysconfig
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_LIBDIR = _PKG / "lib"
_LIBNAME = "libst_pybinding"
_LIB = _LIBDIR / f"{_LIBNAME}.so"
_DIGEST = _LIBDIR / "sources.sha256"

SOURCES = [
    "kernels/gemm_launch.cu",
    "kernels/rmsnorm.cu",
    "kernels/comm_kernels.cu",
    "kernels/no_alloc_entry.cu",
    "runtime/symm_heap.cpp",
    "runtime/engine.cpp",
    "api/nccl_utils.cpp",
    "api/overlap_impl.cpp",
    "api/baseline_impl.cpp",
    "api/bindings.cpp",
]

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def library_path() -> Path:
    return _LIB


def _existing_sources() -> list[Path]:
    """The fixed sources plus one generated file per kernel instance
    (tool/generate_instances.py writes csrc/kernels/generated/)."""
    generated = sorted((_CSRC / "kernels" / "generated").glob("*.cu"))
    return [(_CSRC / s) for s in SOURCES if (_CSRC / s).exists()] + generated


def _source_digest() -> str:
    h = hashlib.sha256()
    files = sorted(p for p in _CSRC.rglob("*") if p.suffix in {".cu", ".cuh", ".cpp", ".h", ".inc"})
    for p in files:
        h.update(str(p.relative_to(_CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(CUDA_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return _LIB.exists() and _DIGEST.exists() and _DIGEST.read_text().strip() == _source_digest()


def _site_packages() -> Path:
    return Path(sysconfig.get_paths()["purelib"])


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and is_current():
        return _LIB
    if shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists():
        raise RuntimeError("flashoverlap_b200: nvcc not found, cannot build the native library")
    os.environ.setdefault("CUDA_HOME", "/usr/local/cuda")
    from torch.utils import cpp_extension

    _LIBDIR.mkdir(exist_ok=True)
    sp = _site_packages()
    nccl = sp / "nvidia" / "nccl"
    cublas = sp / "nvidia" / "cublas"
    include_paths = [str(_CSRC)]
    # Resolve the C++ runtime against the shared libstdc++ explicitly: a compiler
    # wrapper whose own libstdc++.so link is broken would otherwise pull the
    # exception runtime in statically, and a second copy of it in one process
    # crashes as soon as an exception unwinds through this library.
    ldflags = ["-L/usr/lib/x86_64-linux-gnu", "-l:libstdc++.so.6", "-l:libgcc_s.so.1"]
    if (nccl / "include" / "nccl.h").exists():
        include_paths.append(str(nccl / "include"))
        ldflags += [f"-L{nccl / 'lib'}", "-l:libnccl.so.2", f"-Wl,-rpath,{nccl / 'lib'}"]
    else:
        ldflags += ["-lnccl"]
    if (cublas / "lib" / "libcublas.so.12").exists():
        ldflags += [f"-L{cublas / 'lib'}", "-l:libcublas.so.12", f"-Wl,-rpath,{cublas / 'lib'}"]
    else:
        ldflags += ["-lcublas"]
    # A digest left over from an earlier build must not vouch for a library this
    # build fails to replace.
    if _DIGEST.exists():
        _DIGEST.unlink()
    cpp_extension.load(
        name=_LIBNAME,
        sources=[str(p) for p in _existing_sources()],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=CUDA_FLAGS,
        extra_ldflags=ldflags,
        extra_include_paths=include_paths,
        build_directory=str(_LIBDIR),
        is_python_module=False,
        verbose=verbose,
    )
    if not _LIB.exists():
        raise RuntimeError(f"flashoverlap_b200: build finished but {_LIB} is missing")
    newest = max(p.stat().st_mtime for p in _CSRC.rglob("*") if p.suffix in {".cu", ".cuh", ".cpp", ".h", ".inc"})
    if _LIB.stat().st_mtime < newest:
        # (a retry after a failed build in the same process makes torch skip the build and load the old file)
        raise RuntimeError(f"flashoverlap_b200: {_LIB} is older than its sources: the build did not replace it; "
                           "run `python -m flashoverlap_b200._build --force` in a fresh process to see the compiler error")
    _DIGEST.write_text(_source_digest() + "\n")
    return _LIB


_loaded = False


def load(verbose: bool = False) -> Path:
    """Load the native library into this process (building it first if needed)."""
    global _loaded
    if _loaded:
        return _LIB
    import torch

    if not is_current():
        build(verbose=verbose)
    torch.ops.load_library(str(_LIB))
    _loaded = True
    return _LIB


if __name__ == "__main__":
    import sys

    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
