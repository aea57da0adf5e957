"""pip-installable build of the attention path (sm_100a only).

Counterpart of the reference's setup.py (setup.py:19-86 of dsuarez01/minfer-python), which builds
a torch CUDAExtension for compute_89 and asserts a GPU at build time.  Here the native part is a
plain C-ABI shared library, so the build step is one nvcc invocation (build.py) run before the
Python files are collected; no GPU, no torch headers and no other architecture are involved.

    python setup.py build_py        # compiles libminfer_attn.so in-tree, next to the Python binding
    pip install --no-build-isolation -e .
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


class BuildWithNvcc(build_py):
    def run(self):
        import build as native
        native.build()
        super().run()


setup(
    name="minfer-b200-attn",
    version="0.2.0",
    description="B200-native attention path behind minfer's op surface",
    packages=find_packages(include=["minfer", "minfer.*"]),
    package_data={"minfer.kernels.torch_ext": ["libminfer_attn.so"]},
    python_requires=">=3.10",
    cmdclass={"build_py": BuildWithNvcc},
)
