"""``B200Platform``: the out-of-tree vLLM platform class, and the same information for standalone use.

Reference: ``KunlunPlatform`` (``vllm_kunlun/platforms/kunlun.py:22-390``): device identity, capability,
memory query, config fix-ups, attention-backend selection, communicator / punica / graph-wrapper class
paths.  Deliberate differences: total memory is the GPU's (the reference returns host RAM,
``:108-129``); peak-memory statistics are not reset before being read (``:285-306``);
``opaque_attention_op`` is a classmethod (``:366-370`` lacks the decorator)."""
from __future__ import annotations

from typing import Optional

import torch

try:  # the platform class only subclasses vLLM's when vLLM is importable
    from vllm.platforms.interface import Platform as _VllmPlatform
    from vllm.platforms.interface import PlatformEnum as _PlatformEnum
    _HAVE_VLLM = True
except Exception:  # pragma: no cover - vLLM is optional
    _VllmPlatform = object
    _PlatformEnum = None
    _HAVE_VLLM = False


class B200Platform(_VllmPlatform):
    if _HAVE_VLLM:
        _enum = _PlatformEnum.OOT
    device_name: str = "cuda"
    device_type: str = "cuda"
    dispatch_key: str = "CUDA"
    ray_device_key: str = "GPU"
    dist_backend: str = "nccl"
    device_control_env_var: str = "CUDA_VISIBLE_DEVICES"
    simple_compile_backend: str = "eager"
    supported_quantization: list = ["fp8", "compressed-tensors", "awq", "gptq"]
    supported_dtypes = [torch.bfloat16, torch.float16, torch.float32]

    # ---- identity ----
    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        return torch.cuda.get_device_name(device_id) if torch.cuda.is_available() else "NVIDIA B200"

    @classmethod
    def get_device_capability(cls, device_id: int = 0):
        major, minor = torch.cuda.get_device_capability(device_id) if torch.cuda.is_available() else (10, 0)
        if _HAVE_VLLM:
            from vllm.platforms.interface import DeviceCapability
            return DeviceCapability(major=major, minor=minor)
        return (major, minor)

    @classmethod
    def get_device_uuid(cls, device_id: int = 0) -> str:
        return str(torch.cuda.get_device_properties(device_id).uuid) if torch.cuda.is_available() else "cpu"

    @classmethod
    def manual_seed_all(cls, seed: int) -> None:
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    @classmethod
    def num_compute_units(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).multi_processor_count if torch.cuda.is_available() else 148

    @classmethod
    def device_count(cls) -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    @classmethod
    def stateless_init_device_torch_dist_pg(cls, backend, prefix_store, group_rank, group_size, timeout):
        """NCCL process group without the global state of ``init_process_group`` (upstream's CUDA recipe)."""
        from torch.distributed import ProcessGroup
        from torch.distributed.distributed_c10d import ProcessGroupNCCL
        pg = ProcessGroup(prefix_store, group_rank, group_size)
        opts = ProcessGroupNCCL.Options()
        opts._timeout = timeout
        be = ProcessGroupNCCL(prefix_store, group_rank, group_size, opts)
        pg._set_default_backend(ProcessGroup.BackendType.NCCL)
        be._set_sequence_number_for_group()
        pg._register_backend(torch.device("cuda"), ProcessGroup.BackendType.NCCL, be)
        return pg

    @classmethod
    def has_device_capability(cls, capability, device_id: int = 0) -> bool:
        cap = cls.get_device_capability(device_id)
        cap = (cap.major, cap.minor) if hasattr(cap, "major") else tuple(cap)
        want = capability if isinstance(capability, tuple) else (capability // 10, capability % 10)
        return cap >= tuple(want)

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        if torch.cuda.is_available():
            return torch.cuda.get_device_properties(device_id).total_memory
        return 180 * (1 << 30)

    @classmethod
    def get_current_memory_usage(cls, device: Optional[torch.device] = None) -> float:
        return float(torch.cuda.max_memory_allocated(device)) if torch.cuda.is_available() else 0.0

    @classmethod
    def is_async_output_supported(cls, enforce_eager: Optional[bool]) -> bool:
        return True

    @classmethod
    def is_pin_memory_available(cls) -> bool:
        return True

    @classmethod
    def inference_mode(cls):
        return torch.inference_mode()

    @classmethod
    def set_device(cls, device: torch.device) -> None:
        torch.cuda.set_device(device)

    @classmethod
    def is_sleep_mode_available(cls) -> bool:
        return False

    # ---- class paths (the extension points upstream resolves by string) ----
    @classmethod
    def get_device_communicator_cls(cls) -> str:
        # a ``DeviceCommunicatorBase`` subclass with upstream's constructor; the standalone engine uses
        # ``vllm_kunlun_b200.parallel.communicator.DeviceCommunicator`` on the same peer-memory kernels
        return "vllm_kunlun_b200.distributed.b200_communicator.B200Communicator"

    @classmethod
    def get_punica_wrapper(cls) -> str:
        return "vllm_kunlun_b200.lora.punica_vllm.PunicaWrapperB200"

    @classmethod
    def get_attn_backend_cls(cls, selected_backend, attn_selector_config, num_heads=None) -> str:
        """Upstream's selector calls ``(selected_backend, attn_selector_config, num_heads)``; the choice follows
        ``attn_selector_config.use_mla`` / ``use_sparse`` (``platforms/kunlun.py:247-283``)."""
        use_mla = bool(getattr(attn_selector_config, "use_mla", False))
        use_sparse = bool(getattr(attn_selector_config, "use_sparse", False))
        if use_mla and use_sparse:
            return "vllm_kunlun_b200.attention.backends.SparseMLABackend"
        if use_mla:
            return "vllm_kunlun_b200.attention.backends.MLABackend"
        return "vllm_kunlun_b200.attention.backends.GQABackend"

    @classmethod
    def is_cuda_alike(cls) -> bool:
        return True

    @classmethod
    def use_custom_allreduce(cls) -> bool:
        return False  # the peer-memory kernels live in the device communicator, not in upstream's custom all-reduce

    @classmethod
    def import_kernels(cls) -> None:
        """Load the in-tree extension instead of upstream's ``vllm._C`` and register the out-of-tree layers."""
        from ..ops import _ext
        _ext.load(required=False)
        from ..ops.oot_layers import register_oot_layers
        register_oot_layers()

    @classmethod
    def get_static_graph_wrapper_cls(cls) -> str:
        return "vllm_kunlun_b200.compilation.cuda_graph.DecodeGraphs"

    @classmethod
    def support_static_graph_mode(cls) -> bool:
        return True

    @classmethod
    def opaque_attention_op(cls) -> bool:
        return True

    @classmethod
    def support_hybrid_kv_cache(cls) -> bool:
        return True

    @classmethod
    def check_and_update_config(cls, vllm_config) -> None:
        """Block size 16 by default, 64 for MLA / sparse MLA; custom ops all on; no inductor fusion
        (the fix-ups of ``platforms/kunlun.py:147-245`` that still apply on this hardware)."""
        cache = getattr(vllm_config, "cache_config", None)
        model = getattr(vllm_config, "model_config", None)
        if cache is not None:
            use_mla = bool(getattr(model, "use_mla", False)) if model is not None else False
            if use_mla:
                cache.block_size = 64
            elif not getattr(cache, "block_size", None):
                cache.block_size = 16
        comp = getattr(vllm_config, "compilation_config", None)
        if comp is not None:
            if hasattr(comp, "custom_ops") and not comp.custom_ops:
                comp.custom_ops = ["all"]
        par = getattr(vllm_config, "parallel_config", None)
        if par is not None and getattr(par, "worker_cls", "auto") == "auto":
            par.worker_cls = "vllm.v1.worker.gpu_worker.Worker"

    @classmethod
    def check_if_supports_dtype(cls, dtype) -> None:
        if dtype not in (torch.bfloat16, torch.float16, torch.float32, torch.int8, torch.float8_e4m3fn):
            raise ValueError(f"dtype {dtype} is not supported on B200Platform")

    @classmethod
    def pre_register_and_update(cls, parser=None) -> None:
        from .. import quantization  # noqa: F401  (registers fp8 / int8 / awq / gptq methods)
        from ..ops.oot_layers import register_oot_layers
        register_oot_layers()


def register_models_with_vllm() -> int:
    """Nothing is registered with upstream's ``ModelRegistry``: under upstream vLLM the UPSTREAM model files run,
    on this plugin's out-of-tree layers, attention backends and communicator (dense Llama / Qwen models run that way
    in the reference too, ``vllm_kunlun/models/__init__.py:24-31``).  The model classes of this package belong to
    its standalone engine - they are not ``vllm`` model classes (no ``VllmConfig`` constructor, no
    ``IntermediateTensors``), so registering them would replace working upstream entries with classes upstream
    cannot construct.  Returns the number of registered architectures (0)."""
    return 0
