"""MoBA semantics record, field-compatible with the reference's `MoBAConfig`
(reference: src/moba/config.py:20-99).

Only the flags that change what is computed are honoured by the CUDA engine:
`block_size`, `top_k`, `always_select_current`, `top_k_includes_current`.
`tie_break_low_index` is always true on the device (lowest block id wins a tie)
and `pool_masked_only` is accepted and ignored, exactly as in the reference.
"""

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class MoBAConfig:
    """One MoBA attention configuration (frozen: it identifies a result row).

    block_size: key positions per block.
    top_k: blocks attended per query; includes the query's own block when
        `always_select_current and top_k_includes_current` (the default).
    dtype: compute dtype of the attention (informational for the engine; the
        kernels follow the dtype of the tensors they are given).
    """

    block_size: int
    top_k: int
    dtype: torch.dtype = torch.bfloat16
    always_select_current: bool = True
    top_k_includes_current: bool = True
    tie_break_low_index: bool = True
    pool_masked_only: bool = False
    # Not in the reference. `gate_window` = W restricts the blocks a query may select to the W
    # blocks before its own block plus the first `gate_sinks` blocks of its sequence; the gate
    # then costs O(S * (W + sinks)) instead of O(S * num_blocks). None = every past block (the
    # reference's semantics). It changes which blocks are chosen, so results differ from the
    # reference's by design (the test suite's CPU restatement takes the same two parameters).
    gate_window: Optional[int] = None
    gate_sinks: int = 0

    def __post_init__(self) -> None:
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")
        if self.top_k <= 0:
            raise ValueError(f"top_k must be positive, got {self.top_k}")
        if self.gate_window is not None and self.gate_window <= 0:
            raise ValueError(f"gate_window must be positive or None, got {self.gate_window}")
        if self.gate_sinks < 0 or (self.gate_sinks and self.gate_window is None):
            raise ValueError("gate_sinks must not be negative and needs a gate_window")

    def past_blocks_selected(self, num_blocks: int) -> int:
        """Budget of strictly-past blocks per query, clamped to [0, num_blocks]
        (reference: src/moba/config.py:69-84)."""
        take = self.top_k
        if self.always_select_current and self.top_k_includes_current:
            take -= 1
        return max(0, min(take, num_blocks))

    def num_blocks(self, seq_len: int) -> int:
        """ceil(seq_len / block_size); a short tail block is a real block."""
        return -(-seq_len // self.block_size)

    @property
    def slots_per_query(self) -> int:
        """Output slots a query can fill: the past budget plus the own block.

        Equals `top_k` under the defaults. With `top_k_includes_current=False`
        it is `top_k + 1`; the engine sizes its buffers by this number instead
        of truncating to `top_k`.
        """
        seed = 1 if self.always_select_current else 0
        take = self.top_k - (1 if (seed and self.top_k_includes_current) else 0)
        return take + seed
