"""Packaging entry: ``python setup.py build_ext --inplace`` (or ``pip install --no-build-isolation -e .``) compiles
the two native libraries in-tree with ``rannc_b200.build`` -- nvcc for sm_100a only, g++ for the pybind11 core --
and installs ``rannc_b200`` together with the ``pyrannc`` alias package and the ``bin/rl`` launcher shim.

The reference builds its extension through CMake from setup.py (setup.py, CMakeLists.txt); here the build is a
short Python module because there are only two link targets and no third-party sources."""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    # load rannc_b200/build.py by path: importing the package would already need the libraries
    spec = importlib.util.spec_from_file_location("_rannc_b200_build", os.path.join(ROOT, "rannc_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_core()
    mod.build_kernels()


class BuildNative(Command):
    description = "compile _core (pybind11) and _kernels (CUDA, sm_100a) next to the Python sources"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree")]
    boolean_options = ["inplace"]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPyWithNative(build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    name="rannc_b200",
    version="0.1.0",
    description="Automatic model partitioning and training middleware for PyTorch on NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["rannc_b200", "rannc_b200.*", "pyrannc"]),
    package_data={"rannc_b200": ["*.so", "csrc/core/*", "csrc/cuda/*"]},
    scripts=["bin/rl"],
    python_requires=">=3.10",
    install_requires=["torch>=2.6"],
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
)
