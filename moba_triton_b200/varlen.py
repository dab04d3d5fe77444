"""Packed (variable-length) batch boundary (reference: src/moba/varlen.py:33-236).

`validate_cu_seqlens` runs on every call and never reads device memory.
`pack`, `unpack` and `from_nested` build batches: row gathers done by the CUDA
kernels of csrc/varlen.cu through the C ABI (`moba_b200_pack_index`,
`moba_b200_pack_rows`, `moba_b200_unpack_rows`, `moba_b200_seq_meta`). `pack`
and `from_nested` synchronise once, to learn the token total and the longest
sequence; like every other entry point they take CUDA tensors only.
"""

import torch

from moba_triton_b200 import _lib


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


def _row_bytes(x: torch.Tensor) -> int:
    return x.shape[-2] * x.shape[-1] * x.element_size()


def _read_meta(meta: torch.Tensor):
    """(total tokens, longest sequence): the one host synchronisation of a batch build."""
    total, longest = meta.tolist()
    return int(total), int(longest)


def pack(x: torch.Tensor, attention_mask: torch.Tensor):
    """[B,S,H,D] + [B,S] mask (nonzero = real token) -> (packed [1,T,H,D], cu_seqlens
    int32 [B+1] on the device of x, max_seqlen as an int). Kept rows keep their (b, s) order."""
    if x.ndim != 4:
        raise ValueError(f"x must be [B, S, H, D], got {tuple(x.shape)}")
    b, s, h, d = x.shape
    if tuple(attention_mask.shape) != (b, s):
        raise ValueError(
            f"attention_mask must be [B, S] = {(b, s)}, got {tuple(attention_mask.shape)}")
    _lib.require_cuda(x, attention_mask)
    x = x.contiguous()
    mask = attention_mask.to(x.device)
    if mask.dtype not in (torch.bool, torch.uint8, torch.int8, torch.int32, torch.int64):
        mask = mask != 0
    mask = mask.contiguous()
    i32 = dict(device=x.device, dtype=torch.int32)
    dest = torch.empty((b, s), **i32)
    lengths = torch.empty((b,), **i32)
    cu = torch.empty((b + 1,), **i32)
    meta = torch.empty((2,), **i32)
    _lib.call("moba_b200_pack_index", x.device, "pack", _lib.ptr(mask), mask.element_size(), b, s,
              _lib.ptr(dest), _lib.ptr(lengths), _lib.ptr(cu), _lib.ptr(meta))
    total, longest = _read_meta(meta)
    packed = torch.empty((1, total, h, d), device=x.device, dtype=x.dtype)
    if total:
        _lib.call("moba_b200_pack_rows", x.device, "pack", _lib.ptr(x), _lib.ptr(dest), _lib.ptr(cu),
                  _lib.ptr(packed), b, s, _row_bytes(x))
    return packed, cu, longest


def unpack(packed: torch.Tensor, cu_seqlens: torch.Tensor, batch: int, seq_len: int):
    """Inverse of `pack` for sequences stored from position 0: [1,T,H,D] -> [batch,seq_len,H,D],
    padding positions zeroed."""
    if packed.ndim != 4 or packed.shape[0] != 1:
        raise ValueError(f"packed must be [1, T, H, D], got {tuple(packed.shape)}")
    if cu_seqlens.numel() != batch + 1:
        raise ValueError(
            f"cu_seqlens has {cu_seqlens.numel()} entries, expected {batch + 1} for batch {batch}")
    _lib.require_cuda(packed, cu_seqlens)
    _, _, h, d = packed.shape
    packed = packed.contiguous()
    cu = cu_seqlens.to(device=packed.device, dtype=torch.int32).contiguous()
    out = torch.empty((batch, seq_len, h, d), device=packed.device, dtype=packed.dtype)
    _lib.call("moba_b200_unpack_rows", packed.device, "unpack", _lib.ptr(packed), _lib.ptr(cu), _lib.ptr(out),
              batch, seq_len, _row_bytes(packed))
    return out


def from_nested(nt: torch.Tensor):
    """Jagged nested tensor [B, j, H, D] -> (packed, cu_seqlens, max_seqlen). Its values are
    the packed rows already and its offsets are cu_seqlens; only max_seqlen is computed."""
    if not nt.is_nested:
        raise ValueError("from_nested expects a nested tensor")
    values = nt.values()
    if values.ndim != 3:
        raise ValueError(
            f"expected a [B, j, H, D] jagged tensor; its values are {tuple(values.shape)}")
    _lib.require_cuda(values)
    cu = nt.offsets().to(device=values.device, dtype=torch.int32).contiguous()
    meta = torch.empty((2,), device=values.device, dtype=torch.int32)
    _lib.call("moba_b200_seq_meta", values.device, "from_nested", _lib.ptr(cu), cu.numel() - 1, _lib.ptr(meta))
    _, longest = _read_meta(meta)
    return values.contiguous().unsqueeze(0), cu, longest
