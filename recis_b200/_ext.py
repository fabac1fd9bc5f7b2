"""Build and load the native extension in-tree.

The extension is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``). nvcc cross-compiles
without a GPU, so ``build()`` works on a CPU-only machine; the resulting ``.so`` stays inside the package
directory (``recis_b200/_build``) and is loaded from there. A content hash of the sources decides whether a
rebuild is needed, so a copied tree with fresh mtimes does not recompile.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
_BUILD = os.path.join(_HERE, "_build")
_NAME = "_recis_b200_C"
_lock = threading.Lock()
_module = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-Xcompiler", "-fopenmp",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fopenmp", "-Wno-unused-variable", "-Wno-sign-compare"]


def _openmp_ldflags():
    """Link flags for the C++ and OpenMP runtimes, resolved through the compiler instead of assuming a directory. Two things can
    go wrong on a toolchain whose driver is wrapped: ``-fopenmp`` at link time needs libgomp's spec file, which may be missing,
    and without the directory of the shared ``libstdc++`` on the search path the static one is linked, after which C++ exceptions
    thrown in this library (every ``TORCH_CHECK``) no longer unwind cleanly next to libtorch's dynamic one."""
    import shutil
    import subprocess
    # every C++ driver that can be found: a wrapper in front of the real one may not know the real one's library directories
    drivers = []
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), "/usr/bin/g++", "/usr/bin/c++"):
        if cand and cand not in drivers and os.path.exists(cand):
            drivers.append(cand)

    def where(name):
        for cxx in drivers:
            try:
                path = subprocess.run([cxx, f"-print-file-name={name}"], capture_output=True, text=True, check=True).stdout.strip()
            except Exception:
                continue
            if os.path.isabs(path) and os.path.exists(path):
                return path
        return None

    flags = []
    stdcxx = where("libstdc++.so")
    if stdcxx:
        flags.append(f"-L{os.path.dirname(stdcxx)}")
    gomp = where("libgomp.so") or where("libgomp.so.1")
    flags.append(os.path.realpath(gomp) if gomp else "-lgomp")       # the shared object itself: no spec file needed
    return flags


def _sources():
    out = []
    for root, _dirs, files in os.walk(_CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cpp", ".cc")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _all_inputs():
    out = []
    for root, _dirs, files in os.walk(_CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cpp", ".cc", ".h", ".cuh", ".hpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def source_hash() -> str:
    h = hashlib.sha256()
    for p in _all_inputs():
        h.update(os.path.relpath(p, _CSRC).encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def _so_path():
    return os.path.join(_BUILD, _NAME + ".so")


def _stamp_path():
    return os.path.join(_BUILD, "source.sha256")


def is_built() -> bool:
    if not (os.path.exists(_so_path()) and os.path.exists(_stamp_path())):
        return False
    with open(_stamp_path()) as fh:
        return fh.read().strip() == source_hash()


def build(verbose: bool = False):
    """Compile every source under ``csrc`` into one shared object (ninja, parallel)."""
    import torch  # noqa: F401
    from torch.utils import cpp_extension

    os.makedirs(_BUILD, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(max(2, (os.cpu_count() or 4))))
    cpp_extension.load(
        name=_NAME,
        sources=_sources(),
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=_openmp_ldflags(),
        extra_include_paths=[_CSRC],
        build_directory=_BUILD,
        with_cuda=True,
        is_python_module=True,
        verbose=verbose,
    )
    with open(_stamp_path(), "w") as fh:
        fh.write(source_hash())


def load():
    """Return the extension module, building it first when the sources changed."""
    global _module
    if _module is not None:
        return _module
    with _lock:
        if _module is not None:
            return _module
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        if not is_built():
            if os.environ.get("RECIS_B200_NO_BUILD") == "1":
                raise RuntimeError("recis_b200 native extension is not built and RECIS_B200_NO_BUILD=1")
            build(verbose=os.environ.get("RECIS_B200_VERBOSE_BUILD") == "1")
        spec = importlib.util.spec_from_file_location(_NAME, _so_path())
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[_NAME] = mod
        _module = mod
        return mod
