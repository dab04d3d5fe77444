"""Test support shared by the GPU parity tests."""

import torch

from oracle import moba_oracle as orc

# Absolute caps against the float64/float32 oracle stated for this engine:
ATOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}
# The reference's own relative policy (tests/tolerance.py:35-39,145-170 there):
TOLERANCE_FACTOR, TOLERANCE_FLOOR = 2.0, 1e-6


def max_abs_error(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    both_nan = torch.isnan(a) & torch.isnan(b)
    return float(torch.where(both_nan, torch.zeros_like(a), (a - b).abs()).max())


def slots_of(cfg) -> int:
    return cfg.slots_per_query


def oracle_mask(q, k, cfg, cu=None, max_seqlen=None, return_scores=False):
    return orc.selection_mask(q.cpu(), k.cpu(), cfg.block_size, cfg.top_k, cu_seqlens=cu,
                              max_seqlen=max_seqlen, always_current=cfg.always_select_current,
                              includes_current=cfg.top_k_includes_current,
                              return_scores=return_scores)


def near_tie_report(engine_mask, oracle_mask_, scores, mantissa_bits: int):
    """Classifies every query whose selection differs from the oracle's.

    A difference is a *near tie* when the blocks chosen by only one side have
    scores equal to, or one rounding step away from, those chosen only by the
    other side. Returns (differing_queries, not_near_tie_queries).
    """
    em, om = engine_mask.cpu(), oracle_mask_.cpu()
    rows = (em != om).any(dim=-1).nonzero(as_tuple=False)
    bad = 0
    for idx in rows.tolist():
        e, o, s = em[tuple(idx)], om[tuple(idx)], scores[tuple(idx)]
        only_e, only_o = s[e & ~o], s[o & ~e]
        if only_e.numel() != only_o.numel() or only_e.numel() == 0:
            bad += 1
            continue
        step = 2.0 ** (1 - mantissa_bits) * max(float(only_e.abs().max()), float(only_o.abs().max()), 1e-30)
        if float((only_e.sort().values - only_o.sort().values).abs().max()) > step:
            bad += 1
    return rows.shape[0], bad


def oracle_forward(q, k, v, cfg, block_idx, cu=None, causal=True, dout=None, dtype=torch.float64):
    """Sparse oracle in `dtype` on the host with the given routing."""
    return orc.attention_sparse(q.cpu().to(dtype), k.cpu().to(dtype), v.cpu().to(dtype),
                                cfg.block_size, block_idx.cpu(), cu_seqlens=cu, causal=causal,
                                dout=None if dout is None else dout.cpu().to(dtype),
                                compute_dtype=dtype, row_chunk=256)
