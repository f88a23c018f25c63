"""Wheel build: compiles the kernels (nvcc, sm_100a), the host runtime, the Python module and the tools in the
source tree with execution_ucx_b200/_build.py, then packs the package with what was built.

    python -m pip wheel --no-index --no-build-isolation --no-deps -w dist .

The counterpart of the reference's Bazel wheel rule (axon/python/wheel.bzl, axon/python/BUILD.bazel:496-500);
here the build is the same in-tree build that development uses, so a wheel and a checkout run the same binaries.
"""
import importlib.util
from pathlib import Path

from setuptools import Distribution, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


class BuildNativeThenPython(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("_eux_build", ROOT / "execution_ucx_b200" / "_build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_all(verbose=False)
        super().run()


class BinaryDistribution(Distribution):
    def has_ext_modules(self):  # the wheel carries machine code: tag it for this platform and interpreter
        return True


setup(
    packages=find_packages(include=["execution_ucx_b200", "execution_ucx_b200.*"]),
    package_data={"execution_ucx_b200": ["_lib/*", "axon/*.so"]},
    include_package_data=False,
    cmdclass={"build_py": BuildNativeThenPython},
    distclass=BinaryDistribution,
    zip_safe=False,
)
