"""Builds libspyre_b200.so and _C.so in the tree (see build.py) before setuptools collects them as
package data.  The reference builds its extension from setup.py too (setup.py:100-193)."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithKernels(build_py):
    def run(self):
        sys.path.insert(0, HERE)
        import build as kernels  # build.py next to this file

        kernels.build_library()
        kernels.build_extension()
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
