"""``pip install .`` for oslo_b200.

The CUDA (sm_100a) and C++ sources are compiled in-tree by ``oslo_b200/csrc/build.py`` into ``oslo_b200/_lib/*.so`` during the
build step, and the libraries, the sources and the headers ship as package data (the loader rebuilds a missing library from
the shipped sources).  ``OSLO_B200_SKIP_NATIVE_BUILD=1`` skips compilation at install time; without ``nvcc`` only the host
library is built and the GPU kernels are compiled on first use on a machine that has it.
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithNative(build_py):
    def run(self):
        if os.environ.get("OSLO_B200_SKIP_NATIVE_BUILD", "0") != "1":
            sys.path.insert(0, ROOT)
            try:
                from oslo_b200.csrc import build as native

                native.build_cpu()
                try:
                    native.build_cuda()
                except Exception as e:  # no nvcc on this machine: the host library is still useful (CPU ranks, tests)
                    print(f"[oslo_b200] CUDA kernels not built at install time: {e}", file=sys.stderr)
            finally:
                sys.path.pop(0)
        super().run()


def _version():
    scope = {}
    with open(os.path.join(ROOT, "oslo_b200", "__version__.py")) as f:
        exec(f.read(), scope)
    return scope["__version__"]


setup(
    name="oslo_b200",
    version=_version(),
    description="B200-native large-model training framework with the capabilities of EleutherAI/oslo",
    long_description=open(os.path.join(ROOT, "README.md"), encoding="utf-8").read(),
    long_description_content_type="text/markdown",
    packages=find_packages(include=["oslo_b200", "oslo_b200.*"]),
    package_data={"oslo_b200": ["_lib/*.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "csrc/cpu/*.cpp", "csrc/cpu/*.h"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.4", "numpy"],
    extras_require={"hf": ["transformers", "tokenizers"], "serve": ["fastapi", "uvicorn"], "test": ["pytest"]},
    entry_points={"console_scripts": ["oslo-b200-lightseq=oslo_b200.lightseq.cli:main", "oslo-b200-gemm-search=oslo_b200.ops.gemm_algo:main"]},
    cmdclass={"build_py": BuildWithNative},
    zip_safe=False,
)
