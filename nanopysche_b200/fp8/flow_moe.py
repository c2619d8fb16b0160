"""Re-export of ``fp8_flow_moe.flow_moe`` (reference: fp8/flow_moe.py:3-15)."""
from fp8_flow_moe.flow_moe import FP8_BLOCK_SIZE, FP8FlowMoECompute, FP8FlowMoEConfig  # noqa: F401
