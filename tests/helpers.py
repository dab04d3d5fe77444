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
                              return_scores=return_scores, gate_window=cfg.gate_window, gate_sinks=cfg.gate_sinks)


def near_tie_report(engine_mask, oracle_mask_, scores, mantissa_bits: int):
    """Classifies every query whose selection differs from the oracle's.

    A difference is a *near tie* when the blocks chosen by only one side have
    scores one rounding step away from those chosen only by the other side: the
    tensor-core gate rounds a float32 sum, the oracle the exact one. Blocks whose
    rounded scores are *exactly equal* are not a near tie: for those the rule
    "ties go to the lower block id" decides, and a swap is a tie-break bug.
    Returns (differing_queries, not_near_tie_queries).
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
        gap = (only_e.sort().values - only_o.sort().values).abs()
        if float(gap.max()) > step or float(gap.min()) == 0.0:
            bad += 1
    return rows.shape[0], bad


def assert_on_tensor_core_path(shape, hkv, dtype, cfg, cu=None, max_seqlen=None):
    """Fails unless the gate, the forward and the backward of this problem run the
    tcgen05 kernels when the kernel family is left to the library."""
    from moba_triton_b200 import _lib
    old = _lib.set_kernel_path(_lib.PATH_AUTO)
    try:
        prob = _lib.make_problem(shape, hkv, dtype, cfg, cu, max_seqlen)
        lib = _lib.load()
        for stage in (_lib.STAGE_GATE, _lib.STAGE_FWD, _lib.STAGE_BWD):
            got = lib.moba_b200_path_for(prob, stage)
            assert got == _lib.PATH_TCGEN05, f"stage {stage} would run kernel family {got}, not tcgen05"
    finally:
        _lib.set_kernel_path(old)


def oracle_forward(q, k, v, cfg, block_idx, cu=None, causal=True, dout=None, dtype=torch.float64):
    """Sparse oracle in `dtype` on the host with the given routing."""
    return orc.attention_sparse(q.cpu().to(dtype), k.cpu().to(dtype), v.cpu().to(dtype),
                                cfg.block_size, block_idx.cpu(), cu_seqlens=cu, causal=causal,
                                dout=None if dout is None else dout.cpu().to(dtype),
                                compute_dtype=dtype, row_chunk=256)
