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

    `work_items` [n_seq,Hkv,items_per_row,4] (not in the reference) is the dispatch
    list the persistent tensor-core kernels walk: every column, in `order`, cut into
    items of at most `chunk_tiles` tiles of 128 queries -- {block, first tile, tiles,
    dK/dV partial slot | -1 whole column | -2 padding}. An index without it (built by
    hand) runs on the portable kernels only.
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
    work_items: Optional[torch.Tensor] = None
    chunk_tiles: int = 0
    window: Optional[tuple] = None      # (first query row, rows) when the index lists a query window only

    def c_struct(self) -> "_lib.Index":
        items = self.work_items
        return _lib.Index(self.col_nnz.data_ptr(), self.col_offsets.data_ptr(),
                          self.order.data_ptr(), self.row_indices.data_ptr(),
                          self.head_indices.data_ptr(), self.slot_of_pair.data_ptr(),
                          self.row_indices.shape[-1],
                          None if items is None else items.data_ptr(),
                          0 if items is None else items.shape[2], self.chunk_tiles)


def build_csc_from_indices(block_idx: torch.Tensor, num_blocks: int, cfg: MoBAConfig,
                           num_kv_heads: Optional[int] = None, cu_seqlens=None,
                           max_seqlen=None, window: Optional[tuple] = None) -> CSCIndex:
    """Transposes gate output [B,Hq,S,slots] (int32, -1 padded) into a CSCIndex,
    entirely on the device and without a host synchronisation. `window` = (first row,
    rows) lists only those query rows (padded batches): the index of one step of a
    query-chunked call."""
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
    if window is not None and cu_seqlens is not None:
        raise ValueError("a query window needs a padded batch, not a packed one")
    prob = _lib.make_problem((b, s, hq, 64), hkv, torch.bfloat16, cfg, cu_seqlens, max_seqlen, window=window)
    if prob.num_blocks != num_blocks:
        raise ValueError(f"num_blocks {num_blocks} does not match the sequence length ({prob.num_blocks})")
    dev = block_idx.device
    block_idx = block_idx.contiguous()
    cap = group * (rows if window is None else window[1]) * slots
    i32 = dict(device=dev, dtype=torch.int32)
    col_nnz = torch.empty((n_seq, hkv, num_blocks), **i32)
    col_offsets = torch.empty((n_seq, hkv, num_blocks + 1), **i32)
    order = torch.empty((n_seq, hkv, num_blocks), **i32)
    row_indices = torch.empty((n_seq, hkv, cap), **i32)
    head_indices = torch.empty((n_seq, hkv, cap), **i32)
    slot_of_pair = torch.empty((n_seq, hkv, cap), **i32)
    lib = _lib.load()
    per_row = lib.moba_b200_work_items_per_row(prob)
    _lib.check(per_row, "build_csc_from_indices")
    work_items = torch.empty((n_seq, hkv, per_row, 4), **i32)
    nbytes = lib.moba_b200_transpose_scratch_bytes(prob)
    scratch = torch.empty((max(nbytes, 4),), device=dev, dtype=torch.uint8)
    _lib.call("moba_b200_transpose", dev, "build_csc_from_indices",
              prob, _lib.ptr(block_idx), _lib.ptr(cu_seqlens), _lib.ptr(col_nnz), _lib.ptr(col_offsets),
              _lib.ptr(order), _lib.ptr(row_indices), _lib.ptr(head_indices), _lib.ptr(slot_of_pair),
              _lib.ptr(work_items), _lib.ptr(scratch), scratch.numel())
    return CSCIndex(col_nnz, col_offsets, row_indices, head_indices, slot_of_pair, order,
                    num_blocks=num_blocks, max_slots=slots, num_query_heads=hq,
                    cu_seqlens=cu_seqlens, max_seqlen=max_seqlen,
                    work_items=work_items, chunk_tiles=lib.moba_b200_chunk_tiles(prob), window=window)


def build_csc_fused(q: torch.Tensor, k: torch.Tensor, cfg: MoBAConfig, cu_seqlens=None,
                    max_seqlen=None) -> CSCIndex:
    """pool -> gate -> transpose, all on the device (reference: routing.py:430-464)."""
    kbar = pool_blocks(k, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
    block_idx = gate_select(q, kbar, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
    return build_csc_from_indices(block_idx, kbar.shape[2], cfg, num_kv_heads=k.shape[2],
                                  cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)


def csc_to_mask(index: CSCIndex, seq_len: int) -> torch.Tensor:
    """Dense view of an index: bool [B|1, Hq, seq_len, nb], True where the query (row of the
    token axis, head) lists the block (reference: routing.py:564-624, same contract). Test
    support: it synchronises, and it raises ValueError on an index whose offsets do not
    tile its pair arrays.

    Every pair of a (sequence, kv head) row is labelled with its block by searching the row's
    end offsets, so the whole index is expanded with one search and one indexed store."""
    n_seq, hkv, nb = index.col_nnz.shape
    dev = index.col_nnz.device
    ends = index.col_offsets[..., 1:].long()                          # [n_seq, Hkv, nb]
    starts = index.col_offsets[..., :nb].long()
    if not (torch.equal(ends - starts, index.col_nnz.long()) and bool((starts[..., :1] == 0).all())):
        raise ValueError("col_offsets is not the exclusive prefix sum of col_nnz; the index is inconsistent")
    totals = ends[..., -1]                                            # pairs per row
    cap = index.row_indices.shape[-1]
    if int(totals.max()) > cap:
        raise ValueError(f"the index lists {int(totals.max())} pairs in a row that holds {cap}")
    slot = torch.arange(cap, device=dev).expand(n_seq, hkv, cap)
    block = torch.searchsorted(ends.contiguous(), slot.contiguous(), right=True)   # pair -> its block
    live = slot < totals[..., None]
    seq = torch.arange(n_seq, device=dev).view(n_seq, 1, 1).expand(n_seq, hkv, cap)
    batch_row = torch.zeros_like(seq) if index.cu_seqlens is not None else seq
    out = torch.zeros(1 if index.cu_seqlens is not None else n_seq, index.num_query_heads, seq_len, nb,
                      dtype=torch.bool, device=dev)
    out[batch_row[live], index.head_indices.long()[live], index.row_indices.long()[live], block[live]] = True
    return out
