"""Forward: KV-block-major attention into per-slot partials, then the merge
(reference: src/moba/kernels/moba_fwd.py:529-835).

The partials differ from the reference's (m, l, acc) triple: each (query, slot)
holds the already-normalised output of that one block, `part_o`, and its
log2-sum-exp, `part_lse`. The merged output and the global log-sum-exp are the
same quantities. `combine_partials` still accepts the reference's triple.
"""

from typing import Optional

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.device import MIN_BLOCK_SIZE, check_gathered_head_dim
from moba_triton_b200.gqa import head_group_size
from moba_triton_b200.kernels.gating import gate_select
from moba_triton_b200.kernels.pooling import pool_blocks
from moba_triton_b200.kernels.routing import CSCIndex, build_csc_from_indices, build_csc_fused
from moba_triton_b200.varlen import validate_cu_seqlens


def _validate(q, k, v, cfg: MoBAConfig, cu_seqlens=None, max_seqlen=None) -> None:
    """Shape / configuration checks before any launch; reads no device memory
    (reference: moba_fwd.py:733-780, same ValueError wording keys)."""
    if k.shape != v.shape:
        raise ValueError(f"key/value shape mismatch: {tuple(k.shape)}, {tuple(v.shape)}")
    if q.ndim != 4 or k.ndim != 4:
        raise ValueError(f"shape mismatch: expected [B, S, H, D] tensors, got {tuple(q.shape)}, {tuple(k.shape)}")
    if q.shape[0] != k.shape[0] or q.shape[1] != k.shape[1] or q.shape[3] != k.shape[3]:
        raise ValueError(f"shape mismatch: {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError(f"dtype mismatch: {q.dtype}, {k.dtype}, {v.dtype}")
    _lib.dtype_code(q.dtype)
    head_group_size(q.shape[2], k.shape[2])
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"packed input must have batch 1, got {q.shape[0]}; every sequence lives on "
                "the token axis and cu_seqlens says where")
        if max_seqlen is None:
            raise ValueError("max_seqlen is required when cu_seqlens is given")
        validate_cu_seqlens(cu_seqlens, total_tokens=q.shape[1], max_seqlen=max_seqlen)
    ok, reason = check_gathered_head_dim(q.shape[-1], q.element_size())
    if not ok:
        raise ValueError(reason)
    if cfg.block_size < MIN_BLOCK_SIZE:
        raise ValueError(
            f"block_size {cfg.block_size} below the tl.dot minimum of {MIN_BLOCK_SIZE} "
            "(wording kept from the reference; it is this engine's minimum block too)")


def _problem(q, k, cfg, index: CSCIndex, causal=True, part_f32=False):
    """The problem record of a call that uses `index`: the scheduling chunk size is the one
    the index's work items were cut with."""
    return _lib.make_problem(tuple(q.shape), k.shape[2], q.dtype, cfg, index.cu_seqlens,
                             index.max_seqlen, causal=causal, part_f32=part_f32,
                             chunk_tiles=index.chunk_tiles if index.work_items is not None else None,
                             window=index.window)


def _check_index(q, k, cfg, index: CSCIndex) -> None:
    n_seq = index.cu_seqlens.numel() - 1 if index.cu_seqlens is not None else q.shape[0]
    want = (n_seq, k.shape[2], cfg.num_blocks(index.max_seqlen if index.cu_seqlens is not None else q.shape[1]))
    if tuple(index.col_nnz.shape) != want or index.num_query_heads != q.shape[2] \
            or index.max_slots != cfg.slots_per_query:
        raise ValueError(
            f"index mismatch: index covers {tuple(index.col_nnz.shape)} columns, "
            f"{index.num_query_heads} query heads, {index.max_slots} slots; the call needs "
            f"{want}, {q.shape[2]}, {cfg.slots_per_query}")


def empty_partials(shape, slots: int, device, partials_dtype: torch.dtype = torch.float32):
    """Uninitialised (part_lse [B,H,S,slots] f32, part_o [B,H,S,slots,D]) for a
    query of `shape` = (B, S, H, D)."""
    b, s, h, d = shape
    return (torch.empty((b, h, s, slots), device=device, dtype=torch.float32),
            torch.empty((b, h, s, slots, d), device=device, dtype=partials_dtype))


def attend_partials(q, k, v, cfg: MoBAConfig, index: CSCIndex, causal: bool = True,
                    partials_dtype: Optional[torch.dtype] = None, partials=None):
    """Runs the attention stage; returns (part_lse, part_o). `part_lse` is in
    log2 units and -inf where no block wrote the slot; `part_o` of such a slot
    is uninitialised."""
    _lib.require_cuda(q, k, v)
    _check_index(q, k, cfg, index)
    if partials_dtype is None:
        partials_dtype = q.dtype
    if partials_dtype not in (q.dtype, torch.float32):
        raise ValueError(f"partials_dtype must be {q.dtype} or float32, got {partials_dtype}")
    if partials is None:
        rows = q.shape[1] if index.window is None else index.window[1]
        partials = empty_partials((q.shape[0], rows, q.shape[2], q.shape[3]), index.max_slots, q.device, partials_dtype)
    part_lse, part_o = partials
    prob = _problem(q, k, cfg, index, causal, part_o.dtype == torch.float32 and q.dtype != torch.float32)
    ix = index.c_struct()
    _lib.call("moba_b200_fwd", q.device, "attend_partials", prob, _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ix,
              _lib.ptr(index.cu_seqlens), _lib.ptr(part_o), _lib.ptr(part_lse))
    return part_lse, part_o


def merge_partials(part_lse, part_o, out_dtype: torch.dtype, return_lse: bool = False,
                   out=None, lse=None, window=None):
    """LSE merge of (part_lse [B,H,S,K], part_o [B,H,S,K,D]) -> O [B,S,H,D]
    (and lse [B,H,S], log2 units). With `window` = (first row, rows) the partials hold
    that query window only and rows [first, first + rows) of the given `out` (and `lse`)
    are written."""
    _lib.require_cuda(part_lse, part_o)
    b, h, s, slots = part_lse.shape
    d = part_o.shape[-1]
    if tuple(part_o.shape) != (b, h, s, slots, d):
        raise ValueError(f"shape mismatch: part_o {tuple(part_o.shape)} against {(b, h, s, slots, d)}")
    part_lse, part_o = part_lse.contiguous(), part_o.contiguous()
    if window is not None:
        if out is None or s != window[1]:
            raise ValueError("a windowed merge writes into `out`, and the partials hold window[1] rows")
        s = out.shape[1]
    if out is None:
        out = torch.empty((b, s, h, d), device=part_o.device, dtype=out_dtype)
    if lse is None and return_lse:
        lse = torch.empty((b, h, s), device=part_o.device, dtype=torch.float32)
    cfg = MoBAConfig(block_size=16, top_k=slots, always_select_current=False)   # only `slots` matters here
    prob = _lib.make_problem((b, s, h, d), h, out_dtype, cfg,
                             part_f32=part_o.dtype == torch.float32 and out_dtype != torch.float32,
                             window=window)
    if part_o.dtype not in (out_dtype, torch.float32):
        raise ValueError(f"part_o must be {out_dtype} or float32, got {part_o.dtype}")
    _lib.call("moba_b200_merge", out.device, "combine_partials", prob, _lib.ptr(part_o), _lib.ptr(part_lse),
              _lib.ptr(out), _lib.ptr(lse))
    return (out, lse) if return_lse else out


def combine_partials(part_m, part_l, part_acc, out_dtype: torch.dtype, block_m=None,
                     return_lse: bool = False):
    """Reference-signature merge (moba_fwd.py:668-725): takes per-slot maxima,
    denominators and unnormalised accumulators, with `part_m == -inf` marking an
    unwritten slot, and feeds them to the merge kernel as (lse, normalised O)."""
    b, h, s, slots = part_m.shape
    d = part_acc.shape[-1]
    if part_l.shape != part_m.shape:
        raise ValueError(f"shape mismatch: part_l {tuple(part_l.shape)} against part_m {tuple(part_m.shape)}")
    if tuple(part_acc.shape) != (b, h, s, slots, d):
        raise ValueError(f"shape mismatch: part_acc {tuple(part_acc.shape)} against {(b, h, s, slots, d)}")
    written = part_m > float("-inf")
    lse = torch.where(written, part_m + torch.log2(part_l), torch.full_like(part_m, float("-inf")))
    o = torch.where(written[..., None], part_acc.float() / part_l[..., None], torch.zeros((), device=part_m.device))
    return merge_partials(lse, o.contiguous(), out_dtype, return_lse=return_lse)


def query_windows(seq_len: int, query_chunk: int):
    """(first row, rows) of the steps of a query-chunked call."""
    if query_chunk < 1:
        raise ValueError(f"query_chunk must be positive, got {query_chunk}")
    return [(w0, min(query_chunk, seq_len - w0)) for w0 in range(0, seq_len, query_chunk)]


def forward_in_query_chunks(q, k, v, cfg: MoBAConfig, query_chunk: int, causal: bool = True,
                            partials_dtype: Optional[torch.dtype] = None, return_lse: bool = False):
    """The forward run a window of `query_chunk` query rows at a time (padded batches): the
    gate runs once, then every window gets its own index and reuses one set of partial
    buffers of `query_chunk` rows. Every (query, block) pair is computed exactly as in the
    whole call, so the output is the same bit for bit. Returns (out, lse or None, block_idx).
    The reference planned this host-side chunking and never built it
    (docs/deferred-decisions.md:152-220)."""
    b, s, hq, d = q.shape
    kbar = pool_blocks(k, cfg)
    block_idx = gate_select(q, kbar, cfg)
    out = torch.empty_like(q)
    lse = torch.empty((b, hq, s), device=q.device, dtype=torch.float32) if return_lse else None
    partials = None
    for window in query_windows(s, query_chunk):
        index = build_csc_from_indices(block_idx, kbar.shape[2], cfg, num_kv_heads=k.shape[2], window=window)
        if partials is not None and partials[0].shape[2] != window[1]:
            partials = None                                  # the last window may be shorter
        part_lse, part_o = attend_partials(q, k, v, cfg, index, causal=causal, partials_dtype=partials_dtype,
                                           partials=partials)
        partials = (part_lse, part_o)
        merge_partials(part_lse, part_o, q.dtype, return_lse=return_lse, out=out, lse=lse, window=window)
    return out, lse, block_idx


def moba_forward(q, k, v, cfg: MoBAConfig, index: Optional[CSCIndex] = None, causal: bool = True,
                 partials_dtype: Optional[torch.dtype] = None, cu_seqlens=None, max_seqlen=None,
                 kv_heads_per_pass: Optional[int] = None, query_chunk: Optional[int] = None):
    """MoBA attention output [B,S,H,D] in the dtype of q (inference path; no
    log-sum-exp kept). Reference: moba_fwd.py:783-835.

    `kv_heads_per_pass` (not in the reference) runs that many KV heads at a time,
    each with its group of query heads, into one set of partial buffers that every
    pass reuses: same result bit for bit, partial-output memory of one pass.

    `query_chunk` (not in the reference either) runs that many query rows at a time instead:
    the partial buffers then hold `query_chunk` rows, whatever the number of heads. Padded
    batches only; same result bit for bit."""
    if query_chunk is not None:
        if index is not None or kv_heads_per_pass is not None or cu_seqlens is not None:
            raise ValueError("query_chunk cannot be combined with index, kv_heads_per_pass or a packed batch")
        _validate(q, k, v, cfg, None, None)
        _lib.require_cuda(q, k, v)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        return forward_in_query_chunks(q, k, v, cfg, query_chunk, causal, partials_dtype)[0]
    if kv_heads_per_pass is not None:
        if index is not None:
            raise ValueError("kv_heads_per_pass cannot be combined with index (an index spans every head)")
        if kv_heads_per_pass < 1:
            raise ValueError(f"kv_heads_per_pass must be positive, got {kv_heads_per_pass}")
        hkv = k.shape[2]
        if kv_heads_per_pass < hkv:
            group = q.shape[2] // hkv
            out = torch.empty_like(q)
            partials = None
            for h0 in range(0, hkv, kv_heads_per_pass):
                h1 = min(hkv, h0 + kv_heads_per_pass)
                qs = q[:, :, h0 * group:h1 * group].contiguous()
                ks, vs = k[:, :, h0:h1].contiguous(), v[:, :, h0:h1].contiguous()
                _validate(qs, ks, vs, cfg, cu_seqlens, max_seqlen)
                _lib.require_cuda(qs, ks, vs, cu_seqlens)
                idx = build_csc_fused(qs, ks, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
                if partials is not None and partials[1].shape[1] != qs.shape[2]:
                    partials = None                          # the last pass may hold fewer heads
                if partials is None:
                    partials = empty_partials(qs.shape, idx.max_slots, qs.device,
                                              partials_dtype if partials_dtype is not None else q.dtype)
                part_lse, part_o = attend_partials(qs, ks, vs, cfg, idx, causal=causal,
                                                   partials_dtype=partials_dtype, partials=partials)
                out[:, :, h0 * group:h1 * group] = merge_partials(part_lse, part_o, q.dtype)
            return out
    if index is not None:
        cu_seqlens, max_seqlen = index.cu_seqlens, index.max_seqlen
    _validate(q, k, v, cfg, cu_seqlens, max_seqlen)
    _lib.require_cuda(q, k, v, cu_seqlens)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if index is None:
        index = build_csc_fused(q, k, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
    part_lse, part_o = attend_partials(q, k, v, cfg, index, causal=causal, partials_dtype=partials_dtype)
    return merge_partials(part_lse, part_o, q.dtype)
