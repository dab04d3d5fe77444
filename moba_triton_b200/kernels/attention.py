"""The differentiable op (reference: src/moba/kernels/attention.py:53-132)."""

from typing import Optional

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.kernels.moba_bwd import moba_backward
from moba_triton_b200.kernels.moba_fwd import _validate, attend_partials, merge_partials
from moba_triton_b200.kernels.routing import CSCIndex, build_csc_fused


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
                   kv_heads_per_pass: Optional[int] = None) -> torch.Tensor:
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
    heads that is 4.3 GB per pass instead of 34 GB."""
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
