"""Stage 2: per-query block selection (reference: src/moba/kernels/gating.py:343-448)."""

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.gqa import head_group_size
from moba_triton_b200.kernels.pooling import _packed_args


def gate_select(q: torch.Tensor, kbar: torch.Tensor, cfg: MoBAConfig, cu_seqlens=None,
                max_seqlen=None) -> torch.Tensor:
    """q [B,S,Hq,D], kbar [B|n_seq,Hkv,nb,D] -> int32 [B,Hq,S,slots]: the selected
    block ids of every query, ascending, -1 padded, local to the sequence.
    `slots` is `cfg.top_k` under the default flags."""
    _lib.require_cuda(q, kbar, cu_seqlens)
    n_seq = _packed_args(q, cu_seqlens, max_seqlen)
    b, s, h, d = q.shape
    if kbar.ndim != 4 or kbar.shape[0] != n_seq or kbar.shape[-1] != d or kbar.dtype != q.dtype:
        raise ValueError(
            f"representative shape {tuple(kbar.shape)} ({kbar.dtype}) does not match queries "
            f"{tuple(q.shape)} ({q.dtype})")
    head_group_size(h, kbar.shape[1])
    q, kbar = q.contiguous(), kbar.contiguous()
    prob = _lib.make_problem((b, s, h, d), kbar.shape[1], q.dtype, cfg, cu_seqlens, max_seqlen)
    if kbar.shape[2] != prob.num_blocks:
        raise ValueError(
            f"representative shape {tuple(kbar.shape)} does not match {prob.num_blocks} blocks")
    out = torch.empty((b, h, s, prob.slots), device=q.device, dtype=torch.int32)
    _lib.call("moba_b200_gate", q.device, "gate_select", prob, _lib.ptr(q), _lib.ptr(kbar),
              _lib.ptr(cu_seqlens), _lib.ptr(out))
    return out
