"""Packaging (reference: setup.py builds a release wheel around prebuilt CMake libraries).

`python setup.py build_ext --inplace` (or `pip install -e . --no-build-isolation`) compiles the sm_100a kernel library,
the C++ runtime, the example programs and the torch binding IN TREE through csrc/build.py — nvcc cross-compiles without
a GPU — and packages them with the Python sources.
"""
import os
import subprocess
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    subprocess.check_call([sys.executable, os.path.join(ROOT, "csrc", "build.py")])


class BuildExt(Command):
    description = "build libxft_b200_kernels.so / libxft_b200_core.so / libxft_b200_torch.so in tree"
    user_options = [("inplace", "i", "ignored: the libraries are always built in tree"), ("force", "f", "rebuild everything")]
    boolean_options = ["inplace", "force"]

    def initialize_options(self):
        self.inplace = False
        self.force = False

    def finalize_options(self):
        pass

    def run(self):
        cmd = [sys.executable, os.path.join(ROOT, "csrc", "build.py")] + (["--force"] if self.force else [])
        subprocess.check_call(cmd)


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    name="xfastertransformer-b200",
    version="0.3.0",
    description="Blackwell-native (sm_100a) LLM inference engine with the API of xFasterTransformer",
    packages=find_packages(include=["xfastertransformer_b200", "xfastertransformer_b200.*", "xfastertransformer",
                                    "xfastertransformer.*"]),
    package_data={"xfastertransformer_b200": ["lib/*.so", "lib/xft_example", "lib/xft_cb_check", "lib/xft_tp_check"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    extras_require={"convert": ["transformers", "safetensors", "sentencepiece"], "serving": ["grpcio", "fastapi", "uvicorn"]},
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
)
