"""Workload definitions: parameter inventories and layer shapes the fused paths are built and benchmarked for."""
from .deepseek_moe import DEEPSEEK_V3_MOE, KV_REQUEST_BLOCKS, KV_REQUEST_BYTES, MoEConfig  # noqa: F401
from .llama import LLAMA3_8B, LlamaConfig, ParamSpec, param_specs, tp_block  # noqa: F401
