from .llm import LLM, LLMEngine  # noqa: F401
from .request import Request, RequestOutput, SamplingParams  # noqa: F401
