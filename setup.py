"""Packaging: builds the in-tree sm_100a extension and registers the vLLM plugin entry points
(names and groups of the reference: ``setup.py:56-68``)."""
from setuptools import find_packages, setup
from setuptools.command.build_py import build_py


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
    entry_points={
        "vllm.platform_plugins": ["b200 = vllm_kunlun_b200:register"],
        "vllm.general_plugins": [
            "b200_model = vllm_kunlun_b200:register_model",
            "b200_quant = vllm_kunlun_b200:register_quant_method",
            "b200_ops = vllm_kunlun_b200:register_custom_ops",
            "b200_reasoning_parser = vllm_kunlun_b200:register_reasoning_parser",
        ],
        "console_scripts": ["vllm-kunlun-b200 = vllm_kunlun_b200.entrypoints.cli:main"],
    },
)
