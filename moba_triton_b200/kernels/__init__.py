"""Host-side launchers, one module per stage, named after the reference's
`src/moba/kernels/` modules they stand in for:

    pooling   block means            -> moba_b200_pool
    gating    scores + top-k         -> moba_b200_gate
    routing   CSR -> CSC transpose   -> moba_b200_transpose
    moba_fwd  attend + merge         -> moba_b200_fwd, moba_b200_merge
    moba_bwd  delta, dK/dV, dQ       -> moba_b200_bwd
    attention the differentiable op
"""
