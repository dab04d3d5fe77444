"""Stage 3: the KV-block-major index (reference: src/moba/kernels/routing.py:72-624)."""

from dataclasses import dataclass
from typing import Optional

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.gqa import head_group_size
from moba_triton_b200.kernels.gating import gate_select
from moba_triton_b200.kernels.pooling import _packed_args, pool_blocks


@dataclass(frozen=True)
class CSCIndex:
    """Which queries selected each key/value block; field-compatible with the
    reference's `CSCIndex` (routing.py:72-130).

    col_nnz [n_seq,Hkv,nb], col_offsets [n_seq,Hkv,nb+1] (exclusive prefix),
    row_indices / head_indices / slot_of_pair [n_seq,Hkv,G*rows*max_slots]
    (query position -- a packed token index when packed --, absolute query head,
    and which of the query's slots the pair owns), order [n_seq,Hkv,nb] (blocks
    by descending col_nnz, stable). All int32. Unlike the reference, entries of
    a column are always ordered by (query head, position).
    """

    col_nnz: torch.Tensor
    col_offsets: torch.Tensor
    row_indices: torch.Tensor
    head_indices: torch.Tensor
    slot_of_pair: torch.Tensor
    order: torch.Tensor
    num_blocks: int
    max_slots: int
    num_query_heads: int
    cu_seqlens: Optional[torch.Tensor] = None
    max_seqlen: Optional[int] = None

    def c_struct(self) -> "_lib.Index":
        return _lib.Index(self.col_nnz.data_ptr(), self.col_offsets.data_ptr(),
                          self.order.data_ptr(), self.row_indices.data_ptr(),
                          self.head_indices.data_ptr(), self.slot_of_pair.data_ptr(),
                          self.row_indices.shape[-1])


def build_csc_from_indices(block_idx: torch.Tensor, num_blocks: int, cfg: MoBAConfig,
                           num_kv_heads: Optional[int] = None, cu_seqlens=None,
                           max_seqlen=None) -> CSCIndex:
    """Transposes gate output [B,Hq,S,slots] (int32, -1 padded) into a CSCIndex,
    entirely on the device and without a host synchronisation."""
    _lib.require_cuda(block_idx, cu_seqlens)
    b, hq, s, slots = block_idx.shape
    hkv = hq if num_kv_heads is None else num_kv_heads
    group = head_group_size(hq, hkv)
    if cu_seqlens is not None and b != 1:
        raise ValueError(f"packed block ids must have batch 1, got {b}")
    probe = torch.empty((b, s, hq, 0), device="meta")
    n_seq = _packed_args(probe, cu_seqlens, max_seqlen)
    rows = max_seqlen if cu_seqlens is not None else s
    if slots != cfg.slots_per_query:
        raise ValueError(f"block_idx has {slots} slots per query, the configuration {cfg.slots_per_query}")
    # head_dim does not matter to the transpose; 64 keeps the problem record valid
    prob = _lib.make_problem((b, s, hq, 64), hkv, torch.bfloat16, cfg, cu_seqlens, max_seqlen)
    if prob.num_blocks != num_blocks:
        raise ValueError(f"num_blocks {num_blocks} does not match the sequence length ({prob.num_blocks})")
    dev = block_idx.device
    block_idx = block_idx.contiguous()
    cap = group * rows * slots
    i32 = dict(device=dev, dtype=torch.int32)
    col_nnz = torch.empty((n_seq, hkv, num_blocks), **i32)
    col_offsets = torch.empty((n_seq, hkv, num_blocks + 1), **i32)
    order = torch.empty((n_seq, hkv, num_blocks), **i32)
    row_indices = torch.empty((n_seq, hkv, cap), **i32)
    head_indices = torch.empty((n_seq, hkv, cap), **i32)
    slot_of_pair = torch.empty((n_seq, hkv, cap), **i32)
    lib = _lib.load()
    nbytes = lib.moba_b200_transpose_scratch_bytes(prob)
    scratch = torch.empty((max(nbytes, 4),), device=dev, dtype=torch.uint8)
    _lib.call("moba_b200_transpose", dev, "build_csc_from_indices",
              prob, _lib.ptr(block_idx), _lib.ptr(cu_seqlens), _lib.ptr(col_nnz), _lib.ptr(col_offsets),
              _lib.ptr(order), _lib.ptr(row_indices), _lib.ptr(head_indices), _lib.ptr(slot_of_pair),
              _lib.ptr(scratch), scratch.numel())
    return CSCIndex(col_nnz, col_offsets, row_indices, head_indices, slot_of_pair, order,
                    num_blocks=num_blocks, max_slots=slots, num_query_heads=hq,
                    cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)


def build_csc_fused(q: torch.Tensor, k: torch.Tensor, cfg: MoBAConfig, cu_seqlens=None,
                    max_seqlen=None) -> CSCIndex:
    """pool -> gate -> transpose, all on the device (reference: routing.py:430-464)."""
    kbar = pool_blocks(k, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
    block_idx = gate_select(q, kbar, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
    return build_csc_from_indices(block_idx, kbar.shape[2], cfg, num_kv_heads=k.shape[2],
                                  cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)


def csc_to_mask(index: CSCIndex, seq_len: int) -> torch.Tensor:
    """Expands an index to the dense mask [B|1, Hq, seq_len, nb] the oracle uses
    (reference: routing.py:564-624). Test support; synchronises."""
    n_seq, hkv, n = index.col_nnz.shape
    packed = index.cu_seqlens is not None
    dev = index.col_nnz.device
    out = torch.zeros(1 if packed else n_seq, index.num_query_heads, seq_len, n,
                      dtype=torch.bool, device=dev)
    prefix = index.col_nnz.cumsum(-1) - index.col_nnz
    if not torch.equal(prefix.to(index.col_offsets.dtype), index.col_offsets[..., :n]):
        raise ValueError("col_offsets is not the exclusive prefix sum of col_nnz; the index is inconsistent")
    cols = torch.arange(n, device=dev)
    for si in range(n_seq):
        for kv in range(hkv):
            blocks = torch.repeat_interleave(cols, index.col_nnz[si, kv].long())
            total = blocks.numel()
            rows = index.row_indices[si, kv, :total].long()
            heads = index.head_indices[si, kv, :total].long()
            out[0 if packed else si, heads, rows, blocks] = True
    return out
