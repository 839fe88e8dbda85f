"""fp32 CPU oracles for every op (the test ground truth and the timed CPU baseline)."""
from . import attention, basic, misc, moe  # noqa: F401
