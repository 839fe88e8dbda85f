"""Entry points of the package: one table for ``setup.py`` and for the in-tree ``*.egg-info`` that lets the
installed vLLM discover the plugin from a source checkout (names and groups follow the reference's
``setup.py:56-68``)."""
from __future__ import annotations

import os

ENTRY_POINTS = {
    "vllm.platform_plugins": ["b200 = vllm_kunlun_b200:register"],
    "vllm.general_plugins": [
        "b200_model = vllm_kunlun_b200:register_model",
        "b200_quant = vllm_kunlun_b200:register_quant_method",
        "b200_ops = vllm_kunlun_b200:register_custom_ops",
        "b200_reasoning_parser = vllm_kunlun_b200:register_reasoning_parser",
        "b200_tool_parser = vllm_kunlun_b200:register_tool_parser",
    ],
    "console_scripts": ["vllm-kunlun-b200 = vllm_kunlun_b200.entrypoints.cli:main"],
}


def write_egg_info(root: str | None = None) -> str:
    """Write ``<root>/vllm_kunlun_b200.egg-info`` (PKG-INFO + entry_points.txt).  With ``root`` on ``sys.path``
    ``importlib.metadata`` - and therefore ``vllm.plugins.load_plugins_by_group`` - sees the entry points without
    the package being installed."""
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d = os.path.join(root, "vllm_kunlun_b200.egg-info")
    os.makedirs(d, exist_ok=True)
    from .version import __version__
    with open(os.path.join(d, "PKG-INFO"), "w") as fh:
        fh.write(f"Metadata-Version: 2.1\nName: vllm_kunlun_b200\nVersion: {__version__}\n")
    with open(os.path.join(d, "entry_points.txt"), "w") as fh:
        for group, items in ENTRY_POINTS.items():
            fh.write(f"[{group}]\n" + "\n".join(items) + "\n\n")
    with open(os.path.join(d, "top_level.txt"), "w") as fh:
        fh.write("vllm_kunlun_b200\n")
    return d
