"""The differentiable op (reference: src/moba/kernels/attention.py:53-132)."""

from typing import Optional

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.kernels.moba_bwd import moba_backward
from moba_triton_b200.kernels.moba_fwd import (_validate, attend_partials, forward_in_query_chunks,
                                               merge_partials, query_windows)
from moba_triton_b200.kernels.routing import CSCIndex, build_csc_from_indices, build_csc_fused


class MoBAAttentionFunction(torch.autograd.Function):
    """Saves q, k, v, out, the global log2-sum-exp and the per-slot marker; the
    index rides on the context. The gate receives no gradient."""

    @staticmethod
    def forward(ctx, q, k, v, cfg, index, causal, cu_seqlens, max_seqlen):
        if index is not None:
            cu_seqlens, max_seqlen = index.cu_seqlens, index.max_seqlen
        _validate(q, k, v, cfg, cu_seqlens, max_seqlen)
        _lib.require_cuda(q, k, v, cu_seqlens)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        if index is None:
            index = build_csc_fused(q, k, cfg, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
        part_lse, part_o = attend_partials(q, k, v, cfg, index, causal=causal)
        out, lse = merge_partials(part_lse, part_o, q.dtype, return_lse=True)
        ctx.save_for_backward(q, k, v, out, lse, part_lse)
        ctx.cfg, ctx.index, ctx.causal = cfg, index, causal
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, part_lse = ctx.saved_tensors
        dq, dk, dv = moba_backward(dout, q, k, v, out, lse, part_lse, ctx.cfg, ctx.index,
                                   causal=ctx.causal)
        return dq, dk, dv, None, None, None, None, None


class MoBAQueryChunkedFunction(torch.autograd.Function):
    """The op run a window of query rows at a time, forward and backward: the partial
    outputs and dQ partials (slots times the size of the output) exist for one window only.
    Saves the gate's block ids instead of an index; the backward rebuilds each window's
    index from them. O and dQ are the bits of the whole call; dK/dV are summed over the
    windows in float32 and rounded once."""

    @staticmethod
    def forward(ctx, q, k, v, cfg, causal, query_chunk):
        _validate(q, k, v, cfg, None, None)
        _lib.require_cuda(q, k, v)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse, block_idx = forward_in_query_chunks(q, k, v, cfg, query_chunk, causal, return_lse=True)
        ctx.save_for_backward(q, k, v, out, lse, block_idx)
        ctx.cfg, ctx.causal, ctx.query_chunk = cfg, causal, query_chunk
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, block_idx = ctx.saved_tensors
        cfg = ctx.cfg
        nb = cfg.num_blocks(q.shape[1])
        dq = torch.empty_like(q)
        dk32 = torch.zeros(k.shape, device=k.device, dtype=torch.float32)
        dv32 = torch.zeros(v.shape, device=v.device, dtype=torch.float32)
        minus_inf = torch.full((), float("-inf"), device=q.device)
        for window in query_windows(q.shape[1], ctx.query_chunk):
            index = build_csc_from_indices(block_idx, nb, cfg, num_kv_heads=k.shape[2], window=window)
            # which slots of the window's rows were written: those that name a block
            marker = torch.where(block_idx[:, :, window[0]:window[0] + window[1]] >= 0, 0.0, minus_inf).contiguous()
            _, dk_w, dv_w = moba_backward(dout, q, k, v, out, lse, marker, cfg, index, causal=ctx.causal, dq=dq)
            dk32 += dk_w
            dv32 += dv_w
        return dq, dk32.to(k.dtype), dv32.to(v.dtype), None, None, None


def _kv_head_passes(q, k, v, kv_heads_per_pass: int):
    """Slices of (q, k, v) that hold whole groups of query heads with their KV heads."""
    hkv = k.shape[2]
    group = q.shape[2] // hkv
    for h0 in range(0, hkv, kv_heads_per_pass):
        h1 = min(hkv, h0 + kv_heads_per_pass)
        yield q[:, :, h0 * group:h1 * group], k[:, :, h0:h1], v[:, :, h0:h1]


def moba_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: MoBAConfig,
                   index: Optional[CSCIndex] = None, causal: bool = True,
                   cu_seqlens: Optional[torch.Tensor] = None,
                   max_seqlen: Optional[int] = None,
                   kv_heads_per_pass: Optional[int] = None,
                   query_chunk: Optional[int] = None) -> torch.Tensor:
    """MoBA attention with gradient support.

    q [B,S,Hq,D]; k, v [B,S,Hkv,D] with Hkv dividing Hq (grouped-query heads map
    h -> h // (Hq/Hkv)); packed batches are [1,T,H,D] with `cu_seqlens` (int32,
    on the device) and `max_seqlen`. `index` holds routing fixed and carries its
    own packing metadata. `causal=False` removes only the mask inside the
    query's own block. Returns [B,S,Hq,D] in the dtype of q.

    `kv_heads_per_pass` (not in the reference, which planned but never built a
    host-side chunking of the op, docs/deferred-decisions.md:152-220) runs the op
    over that many KV heads at a time, each with its group of query heads. KV
    heads are independent, so the result is the same bit for bit, while the
    per-(query, slot) partial outputs and dQ partials, which are `slots` times the
    size of the output, exist for one pass only: at q [1,524288,32,128] with 8 KV
    heads that is 4.3 GB per pass instead of 34 GB.

    `query_chunk` (the chunking the reference describes there) runs `query_chunk` query
    rows at a time instead, which also bounds the buffers when a GPU holds a single KV
    head. Padded batches only. O and dQ come out bit for bit as from the whole call; dK and
    dV are float32 sums over the windows, rounded once."""
    if query_chunk is not None:
        if index is not None or kv_heads_per_pass is not None or cu_seqlens is not None:
            raise ValueError("query_chunk cannot be combined with index, kv_heads_per_pass or a packed batch")
        return MoBAQueryChunkedFunction.apply(q, k, v, cfg, causal, query_chunk)
    if kv_heads_per_pass is not None:
        if index is not None:
            raise ValueError("kv_heads_per_pass cannot be combined with index (an index spans every head)")
        if kv_heads_per_pass < 1:
            raise ValueError(f"kv_heads_per_pass must be positive, got {kv_heads_per_pass}")
        if kv_heads_per_pass < k.shape[2]:
            outs = [MoBAAttentionFunction.apply(qs, ks, vs, cfg, None, causal, cu_seqlens, max_seqlen)
                    for qs, ks, vs in _kv_head_passes(q, k, v, kv_heads_per_pass)]
            return torch.cat(outs, dim=2)
    return MoBAAttentionFunction.apply(q, k, v, cfg, index, causal, cu_seqlens, max_seqlen)
