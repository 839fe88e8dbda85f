"""Packaging: builds the in-tree sm_100a extension and registers the vLLM plugin entry points
(names and groups of the reference: ``setup.py:56-68``)."""
from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

import importlib.util
import os

_spec = importlib.util.spec_from_file_location(
    "_b200_entry_points", os.path.join(os.path.dirname(os.path.abspath(__file__)), "vllm_kunlun_b200", "_entry_points.py"))
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)
ENTRY_POINTS = _mod.ENTRY_POINTS


class BuildWithKernels(build_py):
    def run(self):
        try:
            from vllm_kunlun_b200.build import build
            build()
        except Exception as e:  # CPU-only installs still get the Python package
            print(f"[vllm_kunlun_b200] CUDA extension not built: {e}")
        super().run()


setup(
    name="vllm_kunlun_b200",
    version="0.1.0",
    description="Blackwell (sm_100a) inference framework with the capabilities of the vLLM-Kunlun plugin",
    packages=find_packages(include=("vllm_kunlun_b200*",)),
    package_data={"vllm_kunlun_b200": ["_C*.so"]},
    python_requires=">=3.10",
    cmdclass={"build_py": BuildWithKernels},
    entry_points=ENTRY_POINTS,
)
