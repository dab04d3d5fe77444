"""Stage 1: mean key per block (reference: src/moba/kernels/pooling.py:103-163)."""

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.varlen import validate_cu_seqlens


def _packed_args(x: torch.Tensor, cu_seqlens, max_seqlen):
    """Common packed-mode checks; returns the sequence count (batch when padded)."""
    if cu_seqlens is None:
        return x.shape[0]
    if x.shape[0] != 1:
        raise ValueError(
            f"packed input must have batch 1, got {x.shape[0]}; every sequence lives on "
            "the token axis and cu_seqlens says where")
    if max_seqlen is None:
        raise ValueError("max_seqlen is required when cu_seqlens is given")
    return validate_cu_seqlens(cu_seqlens, total_tokens=x.shape[1], max_seqlen=max_seqlen)


def pool_blocks(k: torch.Tensor, cfg: MoBAConfig, cu_seqlens=None, max_seqlen=None) -> torch.Tensor:
    """k [B,S,Hkv,D] (or packed [1,T,Hkv,D]) -> block means in the dtype of k:
    [B,Hkv,nb,D] padded, [n_seq,Hkv,cdiv(max_seqlen,bs),D] packed. Rows of a
    short packed sequence are zero past its own block count."""
    _lib.require_cuda(k, cu_seqlens)
    n_seq = _packed_args(k, cu_seqlens, max_seqlen)
    k = k.contiguous()
    b, s, h, d = k.shape
    prob = _lib.make_problem((b, s, h, d), h, k.dtype, cfg, cu_seqlens, max_seqlen)
    out = torch.empty((n_seq, h, prob.num_blocks, d), device=k.device, dtype=k.dtype)
    _lib.call("moba_b200_pool", k.device, "pool_blocks", prob, _lib.ptr(k), _lib.ptr(cu_seqlens), _lib.ptr(out))
    return out
