"""Pins the CPU oracle against vectors produced by the reference's own oracle
(`moba.naive.moba_selection` / `moba_attention_naive`, run in float64 with
autograd gradients). Runs on the host only."""

import torch

from oracle import moba_oracle as orc


def _sel(g, dtype):
    return orc.selection_mask(g.q.to(dtype), g.k.to(dtype), g.block_size, g.top_k,
                              cu_seqlens=g.cu, max_seqlen=g.max_seqlen,
                              always_current=g.always_current,
                              includes_current=g.includes_current)


def test_selection_matches_reference_exactly(golden):
    mask = _sel(golden, golden.low_dtype)
    assert mask.shape == golden.mask.shape
    assert torch.equal(mask, golden.mask)


def test_dense_form_matches_reference_output(golden):
    out = orc.attention_dense(golden.q.double(), golden.k.double(), golden.v.double(),
                              golden.block_size, golden.mask, cu_seqlens=golden.cu)
    live = ~torch.isnan(golden.out)
    assert torch.equal(torch.isnan(out), ~live)
    assert (out[live] - golden.out[live].double()).abs().max() < 2e-6   # stored as float32


def test_sparse_form_matches_reference_output_and_gradients(golden):
    idx = orc.mask_to_block_idx(golden.mask, golden.slots)
    assert torch.equal(orc.block_idx_to_mask(idx, golden.mask.shape[-1]), golden.mask)
    do = golden.do.double() if golden.has_grads else None
    res = orc.attention_sparse(golden.q.double(), golden.k.double(), golden.v.double(),
                               golden.block_size, idx, cu_seqlens=golden.cu, dout=do,
                               compute_dtype=torch.float64, row_chunk=64)
    out = res[0]
    live = ~torch.isnan(golden.out)
    assert torch.equal(torch.isnan(out), ~live)
    assert (out[live] - golden.out[live].double()).abs().max() < 2e-6
    if golden.has_grads:
        for got, want in zip(res[2:], (golden.dq, golden.dk, golden.dv)):
            assert (got - want.double()).abs().max() < 2e-6


def test_low_precision_dense_run_is_close_to_reference_low_precision(golden):
    if golden.out_low is None:
        return
    dt = golden.low_dtype
    out = orc.attention_dense(golden.q.to(dt), golden.k.to(dt), golden.v.to(dt),
                              golden.block_size, golden.mask, cu_seqlens=golden.cu)
    assert (out.float() - golden.out_low.float()).abs().max() <= 2e-2


def test_lse_is_log2_of_the_softmax_denominator():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 64, 1, 32, generator=g, dtype=torch.float64) for _ in range(3))
    mask = orc.selection_mask(q, k, 16, 2)
    idx = orc.mask_to_block_idx(mask, 2)
    _, lse = orc.attention_sparse(q, k, v, 16, idx, compute_dtype=torch.float64)
    pos = torch.arange(64)
    vis = mask[0, 0][:, pos // 16] & (pos.view(-1, 1) >= pos.view(1, -1))
    logits = (q[0, :, 0] @ k[0, :, 0].T) * 32 ** -0.5
    want = torch.logsumexp(logits.masked_fill(~vis, float("-inf")), dim=-1) * orc.LOG2E
    assert (lse[0, 0] - want).abs().max() < 1e-9


def test_pair_count_closed_forms_match_real_masks():
    g = torch.Generator().manual_seed(3)
    for s, bs, tk in [(512, 32, 4), (1000, 64, 4), (2048, 128, 8)]:
        q, k = (torch.randn(1, s, 1, 32, generator=g) for _ in range(2))
        mask = orc.selection_mask(q, k, bs, tk)
        assert int(mask.sum()) == orc.selected_pairs(s, bs, tk)
        pos = torch.arange(s)
        vis = mask[0, 0][:, pos // bs] & (pos.view(-1, 1) >= pos.view(1, -1))
        assert int(vis.sum()) == orc.attended_pairs(s, bs, tk)
