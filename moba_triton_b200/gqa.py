"""Grouped-query head mapping (reference: src/moba/gqa.py:22-84).

Query head `h` reads key/value head `h // group` where
`group = H_q // H_kv`; the group is read off the tensor shapes.
"""

import torch


def head_group_size(num_query_heads: int, num_kv_heads: int) -> int:
    """Returns H_q // H_kv, raising ValueError unless it is a whole number."""
    if num_query_heads <= 0 or num_kv_heads <= 0:
        raise ValueError(
            f"head counts must be positive, got q={num_query_heads} kv={num_kv_heads}"
        )
    if num_query_heads % num_kv_heads:
        raise ValueError(
            f"query heads {num_query_heads} must be divisible by key/value "
            f"heads {num_kv_heads}"
        )
    return num_query_heads // num_kv_heads


def expand_kv(t: torch.Tensor, num_query_heads: int, dim: int = 2) -> torch.Tensor:
    """Test support: repeats each KV head for the query heads sharing it, with
    the copies adjacent (`repeat_interleave`), so head g maps to g // group."""
    group = head_group_size(num_query_heads, t.shape[dim])
    return t if group == 1 else t.repeat_interleave(group, dim=dim)
