"""Packaging of ``oslo_b200`` (the reference ships ``oslo-core`` with sources compiled at first use, setup.py:8-26).

``pip install -e .`` / ``python setup.py build_ext --inplace`` compile the two in-tree extensions ahead of time
through ``oslo_b200.build`` (one target: ``compute_100a/sm_100a``); nothing is compiled at run time.
"""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_extensions() -> None:
    sys.path.insert(0, HERE)
    from oslo_b200 import build as b
    b.build_all(force=False, verbose=True)


class BuildExt(Command):
    description = "compile oslo_b200/_C.so (sm_100a kernels) and oslo_b200/_data_C.so (dataset index builders) in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _build_extensions()


class BuildPy(build_py):
    def run(self):
        _build_extensions()
        super().run()


setup(
    name="oslo-b200",
    version="0.1.0",
    description="Blackwell-native 3D-parallel transformer training and inference framework with OSLO's API",
    packages=find_packages(include=["oslo_b200", "oslo_b200.*"]),
    package_data={"oslo_b200": ["_C.so", "_C_bounds.so", "_data_C.so", "csrc/*"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
)
