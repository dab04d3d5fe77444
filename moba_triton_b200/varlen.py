"""Packed (variable-length) batch boundary (reference: src/moba/varlen.py:33-236).

`validate_cu_seqlens` runs on every call and never reads device memory.
`pack`, `unpack` and `from_nested` build batches and may synchronise once.
"""

import torch
import torch.nn.functional as F


def validate_cu_seqlens(cu_seqlens: torch.Tensor, total_tokens: int,
                        max_seqlen: int, strict: bool = False) -> int:
    """Checks packed metadata, returns the sequence count.

    Rank, length, dtype (int32) and `max_seqlen > 0` are always checked. Value
    checks (starts at 0, strictly increasing, ends at `total_tokens`, longest
    <= `max_seqlen`) run only for a CPU tensor or with `strict=True`, because
    on a device tensor each would be a host synchronisation.
    """
    if cu_seqlens.ndim != 1:
        raise ValueError(f"cu_seqlens must be 1-D, got shape {tuple(cu_seqlens.shape)}")
    if cu_seqlens.numel() < 2:
        raise ValueError(
            f"cu_seqlens needs at least two entries (one sequence), got {cu_seqlens.numel()}")
    if cu_seqlens.dtype != torch.int32:
        raise ValueError(f"cu_seqlens must be int32, got {cu_seqlens.dtype}")
    if max_seqlen is None or max_seqlen <= 0:
        raise ValueError(f"max_seqlen must be positive, got {max_seqlen}")
    if cu_seqlens.device.type == "cpu" or strict:
        cu = cu_seqlens.cpu().tolist()
        if cu[0] != 0:
            raise ValueError(f"cu_seqlens must start at 0, got {cu[0]}")
        lengths = [b - a for a, b in zip(cu[:-1], cu[1:])]
        if min(lengths) <= 0:
            raise ValueError(
                f"cu_seqlens must be strictly increasing (no empty sequence), got lengths {lengths}")
        if cu[-1] != total_tokens:
            raise ValueError(
                f"cu_seqlens ends at {cu[-1]} but the total token count is {total_tokens}")
        if max(lengths) > max_seqlen:
            raise ValueError(
                f"max_seqlen {max_seqlen} is below the longest sequence {max(lengths)}")
    return cu_seqlens.numel() - 1


def pack(x: torch.Tensor, attention_mask: torch.Tensor):
    """[B,S,H,D] + [B,S] mask -> (packed [1,T,H,D], cu_seqlens int32 [B+1], max_seqlen)."""
    if x.ndim != 4:
        raise ValueError(f"x must be [B, S, H, D], got {tuple(x.shape)}")
    b, s = x.shape[:2]
    if tuple(attention_mask.shape) != (b, s):
        raise ValueError(
            f"attention_mask must be [B, S] = {(b, s)}, got {tuple(attention_mask.shape)}")
    keep = attention_mask.bool()
    lengths = keep.sum(dim=1, dtype=torch.int32)
    cu = F.pad(lengths.cumsum(0, dtype=torch.int32), (1, 0))
    longest = int(lengths.max())
    bi, si = keep.nonzero(as_tuple=True)
    return x[bi, si].unsqueeze(0), cu, longest


def unpack(packed: torch.Tensor, cu_seqlens: torch.Tensor, batch: int, seq_len: int):
    """Inverse of `pack`; padding positions come back as zeros."""
    if packed.ndim != 4 or packed.shape[0] != 1:
        raise ValueError(f"packed must be [1, T, H, D], got {tuple(packed.shape)}")
    if cu_seqlens.numel() != batch + 1:
        raise ValueError(
            f"cu_seqlens has {cu_seqlens.numel()} entries, expected {batch + 1} for batch {batch}")
    _, _, h, d = packed.shape
    lengths = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
    keep = torch.arange(seq_len, device=packed.device)[None, :] < lengths[:, None]
    out = packed.new_zeros(batch, seq_len, h, d)
    bi, si = keep.nonzero(as_tuple=True)
    out[bi, si] = packed[0]
    return out


def from_nested(nt: torch.Tensor):
    """Jagged nested tensor [B, j, H, D] -> (packed, cu_seqlens, max_seqlen)."""
    if not nt.is_nested:
        raise ValueError("from_nested expects a nested tensor")
    values = nt.values()
    if values.ndim != 3:
        raise ValueError(
            f"expected a [B, j, H, D] jagged tensor; its values are {tuple(values.shape)}")
    offsets = nt.offsets()
    longest = int((offsets[1:] - offsets[:-1]).max())
    return values.unsqueeze(0).contiguous(), offsets.to(torch.int32), longest
