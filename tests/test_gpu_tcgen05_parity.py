"""Parity of the tcgen05 kernels (bf16/f16, block_size 128, head_dim 64/128)
with the CPU oracle on the cases where a kernel family switch could hide a bug:
packed batches with ragged sequence ends, padded batches whose last block runs
into the next batch row, exact score ties, queries without an own block, the
extra-slot mode, the non-causal own block and float16.

Every test first asserts that the library would run the tensor-core gate,
forward and backward for its problem, so none of them can pass on the portable
kernels. The cases follow tests/test_varlen.py:300-325,383-408,437-468,
tests/test_gate.py:95-120,200-225 and tests/test_backward.py:72-110 of the
reference.

Tolerances: selections exact, or exact up to near ties (never an exact tie);
outputs and gradients within 2e-2 abs of the float64 oracle with the routing
held fixed.
"""

import pytest
import torch

import moba_triton_b200 as moba
from moba_triton_b200 import _lib
from oracle import moba_oracle as orc

from conftest import make_qkv
from helpers import (ATOL, assert_on_tensor_core_path, max_abs_error, near_tie_report,
                     oracle_forward, oracle_mask)

pytestmark = pytest.mark.gpu


def _grads(q, k, v, cfg, do, **kw):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = moba.moba_attention(q, k, v, cfg, **kw)
    out.backward(do)
    return out.detach(), q.grad, k.grad, v.grad


def _check_selection(mask, q, k, cfg, dtype, cu=None, max_seqlen=None):
    want, scores = oracle_mask(q, k, cfg, cu=cu, max_seqlen=max_seqlen, return_scores=True)
    assert mask.shape == want.shape
    differing, bad = near_tie_report(mask, want, scores, 8 if dtype == torch.bfloat16 else 11)
    assert bad == 0, f"{bad} selections differ from the oracle beyond a near tie"
    assert differing <= max(2, 1e-4 * mask.shape[0] * mask.shape[1] * mask.shape[2])


def _check_op(shape, hkv, dtype, cfg, device, cu=None, seed=31, causal=True, check_selection=True):
    """Selection, output and gradients of one problem against the oracle."""
    longest = None if cu is None else max(b - a for a, b in zip(cu[:-1], cu[1:]))
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    assert_on_tensor_core_path(shape, hkv, dtype, cfg, cu_t, longest)
    q, k, v, do = make_qkv(shape, hkv, dtype=dtype, seed=seed, with_do=True)
    qd, kd, vd, dod = (t.to(device) for t in (q, k, v, do))
    cud = None if cu_t is None else cu_t.to(device)
    kw = dict(cu_seqlens=cud, max_seqlen=longest) if cu is not None else {}

    index = moba.build_csc_fused(qd, kd, cfg, **kw)
    mask = moba.csc_to_mask(index, shape[1])
    if check_selection:
        _check_selection(mask, q, k, cfg, dtype, cu_t, longest)
    kbar = moba.pool_blocks(kd, cfg, **kw)
    block_idx = moba.gate_select(qd, kbar, cfg, **kw)
    assert torch.equal(orc.block_idx_to_mask(block_idx.cpu(), mask.shape[-1]), mask.cpu())

    truth = oracle_forward(q, k, v, cfg, block_idx, cu=cu_t, causal=causal, dout=do)
    got = _grads(qd, kd, vd, cfg, dod, index=index, causal=causal)
    for name, g, t in zip(("out", "dq", "dk", "dv"), got, (truth[0], truth[2], truth[3], truth[4])):
        e = max_abs_error(g, t)
        assert e <= ATOL[dtype], f"{name} error {e:.3e} over {ATOL[dtype]:.0e}"
    fwd = moba.moba_forward(qd, kd, vd, cfg, index=index, causal=causal)
    assert torch.equal(fwd.view(torch.int16), got[0].view(torch.int16)), "inference and training outputs differ"
    return (qd, kd, vd, dod), got, index


# ---------------------------------------------------------------------------
# packed batches: blocks cut per sequence, ragged ends, unaligned sequence starts
# ---------------------------------------------------------------------------

PACKS = [
    # head_dim, Hq, Hkv, cu_seqlens
    (64, 4, 4, [0, 384, 513, 1513, 1641, 1841]),        # 384, 129, 1000, 128, 200 tokens
    (128, 4, 2, [0, 384, 513, 1513, 1641, 1841]),
    (64, 4, 2, [0, 300, 428, 1000, 1024]),              # grouped heads, no aligned start but the first
    (128, 2, 2, [0, 300, 428, 1000, 1024]),
]


@pytest.mark.parametrize("d,hq,hkv,cu", PACKS, ids=[f"d{d}-h{hq}kv{hkv}-{len(cu) - 1}seq" for d, hq, hkv, cu in PACKS])
def test_packed_batch_on_tensor_cores(d, hq, hkv, cu, device):
    cfg = moba.MoBAConfig(128, 4)
    shape = (1, cu[-1], hq, d)
    (qd, kd, vd, dod), (out, dq, dk, dv), index = _check_op(shape, hkv, torch.bfloat16, cfg, device, cu=cu)
    # no column reaches past its sequence
    m = moba.csc_to_mask(index, shape[1]).cpu()
    for a, b in zip(cu[:-1], cu[1:]):
        assert not m[0, :, a:b, cfg.num_blocks(b - a):].any()
    # every sequence run alone gives the same bits: the kernels see the same tiles
    for a, b in zip(cu[:-1], cu[1:]):
        assert_on_tensor_core_path((1, b - a, hq, d), hkv, torch.bfloat16, cfg)
        o1, q1, k1, v1 = _grads(qd[:, a:b], kd[:, a:b], vd[:, a:b], cfg, dod[:, a:b])
        assert torch.equal(out[:, a:b], o1), f"packed forward differs from sequence [{a},{b}) run alone"
        assert torch.equal(dq[:, a:b], q1), f"packed dQ differs from sequence [{a},{b}) run alone"
        assert torch.allclose(dk[:, a:b].float(), k1.float(), rtol=2e-2, atol=1e-3)
        assert torch.allclose(dv[:, a:b].float(), v1.float(), rtol=2e-2, atol=1e-3)


@pytest.mark.parametrize("d", [64, 128])
def test_padded_batch_whose_last_block_runs_into_the_next_row(d, device):
    """batch 2, S = 1000: block 7 of row 0 holds 104 tokens and the 24 rows behind it in
    memory belong to batch row 1 (non-zero data that must not be attended)."""
    cfg = moba.MoBAConfig(128, 4)
    _check_op((2, 1000, 4, d), 2, torch.bfloat16, cfg, device, seed=37)


# ---------------------------------------------------------------------------
# exact ties: the lower block id wins, bit for bit
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("top_k", [4, 8])
def test_exact_ties_go_to_the_lower_block_on_tensor_cores(dtype, top_k, device):
    """160 blocks, so the candidates span two chunks of 128 block means: the two halves of
    the selecting warps each hold a list, and the merge of the lists must keep the rule."""
    cfg = moba.MoBAConfig(128, top_k, dtype=dtype)
    nb = 160
    shape = (1, 128 * nb, 2, 64)
    assert_on_tensor_core_path(shape, 2, dtype, cfg)
    q, k, _ = make_qkv(shape, dtype=dtype, seed=2)
    k[:, :, 0] = k[:, :128, 0].repeat(1, nb, 1)             # every block of head 0 is identical
    k[:, 128 * 96:, 1] = k[:, :128 * 64, 1]                 # head 1: blocks 96..159 repeat blocks 0..63
    idx = moba.gate_select(q.to(device), moba.pool_blocks(k.to(device), cfg), cfg).cpu()
    want = orc.mask_to_block_idx(oracle_mask(q, k, cfg), cfg.slots_per_query)
    own = torch.arange(shape[1]) // 128
    late = own >= top_k
    first = torch.arange(top_k - 1, dtype=torch.int32)
    assert torch.equal(idx[0, 0, late, :top_k - 1], first.expand(int(late.sum()), top_k - 1))
    assert torch.equal(idx[0, 0], want[0, 0]), "the tensor-core gate must break exact ties like the oracle"
    # head 1 mixes exact ties (block j and block j + 96) with ordinary scores: a float32 sum that
    # rounds across a boundary may move a pair of equal blocks together, never split the rule
    mask, (om, scores) = orc.block_idx_to_mask(idx, nb), oracle_mask(q, k, cfg, return_scores=True)
    differing, bad = near_tie_report(mask, om, scores, 8 if dtype == torch.bfloat16 else 11)
    assert bad == 0 and differing <= 4, (differing, bad)


# ---------------------------------------------------------------------------
# non-default semantics flags
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("d", [64, 128])
def test_without_own_block_empty_columns_get_exact_zeros(d, device):
    cfg = moba.MoBAConfig(128, 4, always_select_current=False)
    shape = (1, 2048, 4, d)
    (qd, kd, vd, dod), (out, dq, dk, dv), index = _check_op(shape, 2, torch.bfloat16, cfg, device, seed=4)
    empty = (index.col_nnz == 0).nonzero().tolist()
    assert empty, "no unselected block, nothing is being checked"
    for _, h, blk in empty:
        assert not dk[0, blk * 128:(blk + 1) * 128, h].any()
        assert not dv[0, blk * 128:(blk + 1) * 128, h].any()
    assert bool(torch.isnan(out[0, :128].float()).all()), "queries of the first block attend nothing"
    assert not dq[0, :128].any()


@pytest.mark.parametrize("top_k", [2, 8])
def test_extra_slot_mode_on_tensor_cores(top_k, device):
    cfg = moba.MoBAConfig(128, top_k, top_k_includes_current=False)
    assert cfg.slots_per_query == top_k + 1
    _check_op((1, 2048, 2, 64), 2, torch.bfloat16, cfg, device, seed=21)


@pytest.mark.parametrize("d", [64, 128])
def test_non_causal_own_block_on_tensor_cores(d, device):
    cfg = moba.MoBAConfig(128, 3)
    _check_op((1, 1000, 2, d), 2, torch.bfloat16, cfg, device, seed=17, causal=False)
    _check_op((1, 1664, 2, d), 1, torch.bfloat16, cfg, device, cu=[0, 640, 1000, 1664], seed=18, causal=False)


@pytest.mark.parametrize("d", [64, 128])
def test_float16_on_tensor_cores(d, device):
    cfg = moba.MoBAConfig(128, 8, dtype=torch.float16)
    _check_op((1, 2048, 4, d), 2, torch.float16, cfg, device, seed=11)


# ---------------------------------------------------------------------------
# the scheduler's column splitting
# ---------------------------------------------------------------------------

@pytest.fixture
def tiny_chunks():
    old = _lib.set_chunk_tiles(1)                      # every column of two or more tiles is cut
    yield
    _lib.set_chunk_tiles(old)


def _work_item_invariants(index):
    nnz = index.col_nnz.cpu()
    items = index.work_items.cpu()
    n_seq, hkv, nb = nnz.shape
    slots_seen = set()
    for si in range(n_seq):
        for h in range(hkv):
            it = items[si, h]
            it = it[it[:, 3] != -2]                        # drop the padding
            covered = torch.zeros(nb, dtype=torch.int64)
            for blk, tile0, tiles, slot in it.tolist():
                total = -(-int(nnz[si, h, blk]) // 128)
                assert tile0 == covered[blk], "the items of a column must follow one another"
                covered[blk] += tiles
                assert tiles <= index.chunk_tiles and (tiles > 0 or total == 0)
                if slot >= 0:
                    assert total > index.chunk_tiles and slot not in slots_seen
                    slots_seen.add(slot)
                else:
                    assert total <= index.chunk_tiles
            assert torch.equal(covered, -(-nnz[si, h].long() // 128)), "every tile of every column exactly once"
            # dispatch order: heaviest column first, and the list as a whole sorted by size
            first_items = it[it[:, 1] == 0][:, 0].long()
            assert torch.equal(first_items, index.order[si, h].cpu().long())
            assert bool((it[:-1, 2] >= it[1:, 2]).all()), "work items must be listed largest first"
    return len(slots_seen)


def test_work_items_are_listed_largest_first(device):
    """Columns cut at three tiles: pieces of three tiles lead the list, the shorter last pieces
    are merged by size into the uncut columns (the kernels deal the list out in alternating
    direction, which balances a sorted list)."""
    old = _lib.set_chunk_tiles(3)
    try:
        cfg = moba.MoBAConfig(128, 4)
        g = torch.Generator().manual_seed(77)
        q = torch.randn((1, 4096, 4, 64), generator=g).to(torch.bfloat16).to(device)
        k = torch.randn((1, 4096, 2, 64), generator=g).to(torch.bfloat16).to(device)
        index = moba.build_csc_fused(q, k, cfg)
        assert index.chunk_tiles == 3
        assert _work_item_invariants(index) > 0
        items = index.work_items.cpu()[0, 0]
        items = items[items[:, 3] != -2]
        sizes = items[:, 2].tolist()
        assert sizes[0] == 3 and 0 < min(s for s in sizes if s) < 3, "the case must hold pieces of several sizes"
    finally:
        _lib.set_chunk_tiles(old)


@pytest.mark.parametrize("d,hq,hkv,cu", [(64, 4, 2, None), (128, 4, 1, None), (64, 4, 2, [0, 640, 1000, 1664])],
                         ids=["d64", "d128-gqa4", "d64-packed"])
def test_split_columns_give_the_same_results(d, hq, hkv, cu, device, tiny_chunks):
    """With one-tile work items every crowded column is split: forward partials and dQ do not
    depend on the cut (bitwise equal to the unsplit run), dK/dV are sums of float32 partials
    (equal to the oracle within tolerance, and the same bits on every run)."""
    cfg = moba.MoBAConfig(128, 4)
    t = 2048 if cu is None else cu[-1]
    shape = (1, t, hq, d)
    (qd, kd, vd, dod), got, index = _check_op(shape, hkv, torch.bfloat16, cfg, device, cu=cu, seed=51)
    assert index.chunk_tiles == 1
    assert _work_item_invariants(index) > 0, "no column was split, nothing is being checked"
    kw = {} if cu is None else dict(cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=device),
                                    max_seqlen=max(b - a for a, b in zip(cu[:-1], cu[1:])))
    again = _grads(qd, kd, vd, cfg, dod, index=index)
    for a, b in zip(got, again):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), "split runs must be reproducible"
    old = _lib.set_chunk_tiles(1 << 20)                # no column is that long: nothing is cut
    try:
        whole_index = moba.build_csc_fused(qd, kd, cfg, **kw)
        assert _work_item_invariants(whole_index) == 0
        whole = _grads(qd, kd, vd, cfg, dod, index=whole_index)
    finally:
        _lib.set_chunk_tiles(old)
    assert torch.equal(got[0], whole[0]) and torch.equal(got[1], whole[1])
    assert torch.allclose(got[2].float(), whole[2].float(), rtol=2e-2, atol=2e-3)
    assert torch.allclose(got[3].float(), whole[3].float(), rtol=2e-2, atol=2e-3)


# ---------------------------------------------------------------------------
# the candidate-window gate (an extension: bounds the gate's cost; not the reference's semantics)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("window,sinks", [(4, 0), (4, 2), (130, 1), (1, 0), (40, 150), (100000, 0)])
def test_candidate_window_gate_selects_by_the_stated_rule(window, sinks, device):
    """300 blocks, so the recent window and the sinks fall into different 128-block chunks
    and the chunks between them are skipped. The selection is compared with the CPU
    restatement of the same rule; a window wider than the sequence is the unrestricted gate."""
    nb = 300
    shape = (1, 128 * nb, 2, 64)
    cfg = moba.MoBAConfig(128, 8, gate_window=window, gate_sinks=sinks)
    assert_on_tensor_core_path(shape, 1, torch.bfloat16, cfg)
    q, k, _ = make_qkv(shape, 1, dtype=torch.bfloat16, seed=61)
    qd, kd = q.to(device), k.to(device)
    idx = moba.gate_select(qd, moba.pool_blocks(kd, cfg), cfg).cpu()
    mask = orc.block_idx_to_mask(idx, nb)
    _check_selection(mask, q, k, cfg, torch.bfloat16)
    own = (torch.arange(shape[1]) // 128).view(1, 1, -1, 1)
    blocks = torch.arange(nb).view(1, 1, 1, -1)
    allowed = (blocks == own) | ((blocks < own) & ((blocks < sinks) | (blocks >= own - window)))
    assert not (mask & ~allowed).any(), "a block outside the candidate window was selected"
    if window >= nb:
        plain = moba.gate_select(qd, moba.pool_blocks(kd, cfg), moba.MoBAConfig(128, 8)).cpu()
        assert torch.equal(idx, plain)


def test_candidate_window_through_the_whole_op(device):
    cfg = moba.MoBAConfig(128, 4, gate_window=3, gate_sinks=1)
    _check_op((1, 2048, 4, 64), 2, torch.bfloat16, cfg, device, seed=63)
    _check_op((1, 1841, 4, 128), 2, torch.bfloat16, cfg, device, cu=[0, 384, 513, 1513, 1641, 1841], seed=64)
