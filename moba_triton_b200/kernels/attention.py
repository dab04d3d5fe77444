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


def moba_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: MoBAConfig,
                   index: Optional[CSCIndex] = None, causal: bool = True,
                   cu_seqlens: Optional[torch.Tensor] = None,
                   max_seqlen: Optional[int] = None) -> torch.Tensor:
    """MoBA attention with gradient support.

    q [B,S,Hq,D]; k, v [B,S,Hkv,D] with Hkv dividing Hq (grouped-query heads map
    h -> h // (Hq/Hkv)); packed batches are [1,T,H,D] with `cu_seqlens` (int32,
    on the device) and `max_seqlen`. `index` holds routing fixed and carries its
    own packing metadata. `causal=False` removes only the mask inside the
    query's own block. Returns [B,S,Hq,D] in the dtype of q."""
    return MoBAAttentionFunction.apply(q, k, v, cfg, index, causal, cu_seqlens, max_seqlen)
