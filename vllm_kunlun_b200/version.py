"""Version pins (the reference pins upstream vLLM 0.15.1, ``vllm_kunlun/platforms/version.py:3``)."""
__version__ = "0.1.0"
TESTED_VLLM = "0.22.0"
