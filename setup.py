"""python setup.py build_ext --inplace   (or: pip install --no-build-isolation -e .)
Builds the sm_100a extension in place with the package's own build script (nvcc per source file, no torch headers in the
kernels) and installs the pure-Python package.  (reference: setup.py, onmt/modules/extensions/setup.py)"""
import os
import sys

from setuptools import Command, find_packages, setup

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildKernels(Command):
    description = "compile nmtgminor_b200/ops/csrc for sm_100a into nmtgminor_b200/ops/_nmtg_b200_C.so"
    user_options = [("inplace", "i", "accepted for compatibility: the extension is always built in the source tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        sys.path.insert(0, HERE)
        from nmtgminor_b200.ops.build import build
        build()


setup(name="nmtgminor_b200", version="0.2", description="Neural machine / speech translation toolkit for NVIDIA B200 (sm_100a)",
      packages=find_packages(include=["nmtgminor_b200", "nmtgminor_b200.*"]),
      package_data={"nmtgminor_b200.ops": ["csrc/*", "_nmtg_b200_C.so"]},
      cmdclass={"build_ext": BuildKernels, "build_kernels": BuildKernels}, python_requires=">=3.10")
