"""Multi-adapter LoRA serving: Punica-style batched kernels, layer wrappers and the adapter manager."""
from .manager import LoRAManager, LoRARequest  # noqa: F401
from .punica import PunicaWrapperB200  # noqa: F401
