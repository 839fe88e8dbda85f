"""Tool-call parsers (``"glm47"`` as in the reference, ``glm47_moe_tool_parser.py:264``)."""
from .glm47 import Glm47Scanner, Glm47ToolParser  # noqa: F401

TOOL_PARSERS = {"glm47": Glm47ToolParser}
