"""Packaging of recis_b200.

``pip install --no-build-isolation .`` (or ``python setup.py build_ext --inplace``) compiles the native extension for sm_100a
with the same in-tree builder the package uses at import time (``recis_b200/_ext.py``: nvcc + ninja through
``torch.utils.cpp_extension``, ``-gencode arch=compute_100a,code=sm_100a``) and ships the resulting shared objects together
with the C++/CUDA sources, so an installed copy can also rebuild itself after a toolkit change. nvcc cross-compiles without a
GPU; the optional columnar reader needs pyarrow's bundled Arrow headers and is skipped where they are missing.
"""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    sys.path.insert(0, ROOT)
    from recis_b200 import _ext, _ext_io

    if not _ext.is_built():
        _ext.build(verbose=True)
    _ext_io.load()          # builds the reader when it can; returns None otherwise


class BuildNative(Command):
    description = "compile the sm_100a extension in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPyWithNative(build_py):
    def run(self):
        if os.environ.get("RECIS_B200_SKIP_NATIVE_BUILD") != "1":
            _build_native()
        super().run()


setup(
    packages=find_packages(include=["recis_b200", "recis_b200.*"]),
    package_data={"recis_b200": [
        "_build/*.so", "_build/source.sha256", "_build_io/*.so", "_build_io/*.sha256",
        "csrc/*/*.cu", "csrc/*/*.cuh", "csrc/*/*.h", "csrc/*/*.cpp", "csrc/*/*.cc", "csrc_io/*.cpp",
    ]},
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
    zip_safe=False,
)
