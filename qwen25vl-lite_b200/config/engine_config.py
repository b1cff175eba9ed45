"""Scheduling and memory settings of one engine instance.

Names and meanings follow the reference's ``EngineConfig``
(src/qwen25vl_lite/engine.py:43-93) for the options this engine has: ``num_blocks``,
``block_size``, ``max_num_seqs``, ``max_num_batched_tokens``, ``max_model_len``,
``enable_chunked_prefill``, ``dtype``.  One meaning differs and is stated here: the token
budget of a step counts decoded tokens too (one each), because a step is one batch; the
reference's budget counts prompt tokens only (engine.py:631-663).
"""

from __future__ import annotations

from dataclasses import dataclass

DTYPES = ("float32", "bfloat16")


@dataclass
class EngineConfig:
    num_blocks: int = 2048             # pages of each cache group
    block_size: int = 16               # tokens in a page
    max_num_seqs: int = 8              # live requests = per-request state slots
    max_num_batched_tokens: int = 4096  # tokens in one step
    max_model_len: int = 32768         # prompt + generated tokens of one request
    enable_chunked_prefill: bool = True
    dtype: str = "float32"
    cuda_graph: bool = True            # replay decode-only steps from captured graphs
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if self.block_size <= 0 or self.num_blocks <= 0:
            raise ValueError("block_size and num_blocks must be positive")
        if self.max_num_seqs <= 0:
            raise ValueError("max_num_seqs must be positive")
        if self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.max_model_len <= 0:
            raise ValueError("max_model_len must be positive")
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
