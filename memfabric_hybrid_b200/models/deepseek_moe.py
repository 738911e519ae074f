"""Workload shapes of the DeepSeek-V3-style expert-parallel MoE layer and of the DeepSeek-R1 KV-cache block transfer."""
from dataclasses import dataclass


@dataclass(frozen=True)
class MoEConfig:
    hidden: int = 7168
    experts: int = 256
    topk: int = 8
    inter: int = 2048
    act_block: int = 128      # activations: one scale per 1 x 128
    weight_block: int = 128   # weights: one scale per 128 x 128


DEEPSEEK_V3_MOE = MoEConfig()

# One request's KV cache as the reference's latency figure defines it: 61 blocks of 128 KiB and 61 of 16 KiB.
KV_REQUEST_BLOCKS = [128 * 1024] * 61 + [16 * 1024] * 61
KV_REQUEST_BYTES = sum(KV_REQUEST_BLOCKS)
