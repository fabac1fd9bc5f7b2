"""Build and load the native columnar reader (``csrc_io/columnar_reader.cpp``).

It links against the Arrow C++ library that ships inside the installed ``pyarrow`` wheel (headers under
``pyarrow.get_include()``), so it is kept apart from the main extension: where pyarrow or its headers are missing the
reader is simply unavailable (``load()`` returns ``None``) and ``io.OrcDataset`` falls back to its pyarrow-in-Python path.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "csrc_io", "columnar_reader.cpp")
_BUILD = os.path.join(_HERE, "_build_io")
_NAME = "_recis_b200_io"
_lock = threading.Lock()
_module = None
_failed = False


def _arrow():
    import pyarrow as pa
    inc = pa.get_include()
    libdir = pa.get_library_dirs()[0]
    libs = sorted(f for f in os.listdir(libdir) if f.startswith("libarrow.so"))
    pq = sorted(f for f in os.listdir(libdir) if f.startswith("libparquet.so"))
    if not libs or not pq or not os.path.exists(os.path.join(inc, "arrow", "adapters", "orc", "adapter.h")) or not os.path.exists(
            os.path.join(inc, "parquet", "arrow", "reader.h")):
        raise RuntimeError("pyarrow ships no Arrow C++ headers / libraries here")
    return inc, libdir, [libs[-1], pq[-1]]


def _hash():
    h = hashlib.sha256()
    for p in (_SRC, os.path.join(_HERE, "csrc", "common", "rb_hash.cuh")):
        with open(p, "rb") as fh:
            h.update(fh.read())
    try:
        import pyarrow as pa
        h.update(pa.__version__.encode())
    except Exception:
        pass
    return h.hexdigest()


def _so():
    return os.path.join(_BUILD, _NAME + ".so")


def is_built() -> bool:
    stamp = os.path.join(_BUILD, "source.sha256")
    return os.path.exists(_so()) and os.path.exists(stamp) and open(stamp).read().strip() == _hash()


def _stdcxx_dir():
    """The directory of the shared libstdc++ (so that it, not a static copy, is linked): same lookup as the main extension."""
    from . import _ext
    return [f for f in _ext._openmp_ldflags() if f.startswith("-L")]


def build(verbose: bool = False):
    import torch  # noqa: F401
    from torch.utils import cpp_extension
    inc, libdir, libs = _arrow()
    os.makedirs(_BUILD, exist_ok=True)
    cpp_extension.load(
        name=_NAME, sources=[_SRC], extra_cflags=["-O2", "-std=c++20", "-Wno-sign-compare", "-Wno-deprecated-declarations"],
        extra_ldflags=_stdcxx_dir() + [f"-L{libdir}"] + [f"-l:{lib}" for lib in libs] + [f"-Wl,-rpath,{libdir}"],
        extra_include_paths=[inc, "/usr/local/cuda/include"], build_directory=_BUILD, with_cuda=False, is_python_module=True, verbose=verbose)
    with open(os.path.join(_BUILD, "source.sha256"), "w") as fh:
        fh.write(_hash())


def load():
    """The reader module, or ``None`` where it cannot be built (no pyarrow C++ development files)."""
    global _module, _failed
    if _module is not None or _failed:
        return _module
    with _lock:
        if _module is not None or _failed:
            return _module
        try:
            import pyarrow  # noqa: F401  (libarrow must be loaded before the extension resolves its symbols)
            import torch  # noqa: F401
            if not is_built():
                if os.environ.get("RECIS_B200_NO_BUILD") == "1":
                    raise RuntimeError("not built")
                build(verbose=os.environ.get("RECIS_B200_VERBOSE_BUILD") == "1")
            spec = importlib.util.spec_from_file_location(_NAME, _so())
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            sys.modules[_NAME] = mod
            _module = mod
        except Exception as e:                      # noqa: BLE001 - any failure means "reader unavailable"
            _failed = True
            if os.environ.get("RECIS_B200_VERBOSE_BUILD") == "1":
                print(f"native columnar reader unavailable: {e}", file=sys.stderr)
        return _module
