"""Parameter inventory of Llama-style decoders and their tensor-parallel split rules (used by the weight reshard)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


@dataclass(frozen=True)
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


LLAMA3_8B = LlamaConfig()


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: Tuple[int, ...]  # (out, in) for linears, (n,) for norms
    split: str              # "col": split dim 0 over TP (column-parallel), "row": split dim 1 (row-parallel),
                            # "vocab": split dim 0 (vocab-parallel), "rep": replicated
    quantizable: bool       # 2-D linear weights may be cast to fp8 with 128x128 block scales

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def param_specs(cfg: LlamaConfig = LLAMA3_8B) -> List[ParamSpec]:
    """All parameters in a fixed order (embedding, every layer, final norm, lm_head)."""
    h, kvd = cfg.hidden, cfg.kv_heads * cfg.head_dim
    out = [ParamSpec("embed_tokens", (cfg.vocab, h), "vocab", False)]
    for i in range(cfg.layers):
        p = f"layers.{i}."
        out += [
            ParamSpec(p + "input_layernorm", (h,), "rep", False),
            ParamSpec(p + "q_proj", (h, h), "col", True),
            ParamSpec(p + "k_proj", (kvd, h), "col", True),
            ParamSpec(p + "v_proj", (kvd, h), "col", True),
            ParamSpec(p + "o_proj", (h, h), "row", True),
            ParamSpec(p + "post_attention_layernorm", (h,), "rep", False),
            ParamSpec(p + "gate_proj", (cfg.ffn, h), "col", True),
            ParamSpec(p + "up_proj", (cfg.ffn, h), "col", True),
            ParamSpec(p + "down_proj", (h, cfg.ffn), "row", True),
        ]
    out += [ParamSpec("norm", (h,), "rep", False), ParamSpec("lm_head", (cfg.vocab, h), "vocab", False)]
    return out


def tp_block(spec: ParamSpec, tp_rank: int, tp_size: int):
    """(r0, c0, nrows, ncols, cols_full) of the sub-block of `spec` that tensor-parallel rank `tp_rank` holds."""
    if len(spec.shape) == 1:
        return 0, 0, 1, spec.shape[0], spec.shape[0]
    rows, cols = spec.shape
    if spec.split in ("col", "vocab"):
        n = rows // tp_size
        return tp_rank * n, 0, n, cols, cols
    if spec.split == "row":
        n = cols // tp_size
        return 0, tp_rank * n, rows, n, cols
    return 0, 0, rows, cols, cols
