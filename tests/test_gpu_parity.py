"""Parity of the CUDA engine with the CPU oracle and the reference-generated
golden vectors. Every call goes through the public Python API, which is a thin
ctypes layer over the C ABI in include/moba_b200.h.

Tolerances: selections exact (portable gate) or exact up to near ties (tensor
core gate); outputs and gradients within 1e-5 abs for float32 and 2e-2 abs for
bfloat16/float16 of the float64 oracle, and within the reference's relative
policy max(2 x same-dtype-oracle error, 1e-6) where a same-dtype run exists.
"""

import dataclasses

import pytest
import torch

import moba_triton_b200 as moba
from moba_triton_b200 import _lib
from oracle import moba_oracle as orc

from conftest import make_qkv
from helpers import (ATOL, TOLERANCE_FACTOR, TOLERANCE_FLOOR, max_abs_error, near_tie_report,
                     oracle_forward, oracle_mask)

pytestmark = pytest.mark.gpu

PATHS = [pytest.param(_lib.PATH_PORTABLE, id="portable"), pytest.param(_lib.PATH_AUTO, id="auto")]


@pytest.fixture(params=PATHS)
def kernel_path(request):
    old = _lib.set_kernel_path(request.param)
    yield request.param
    _lib.set_kernel_path(old)


def _dev(*ts, device):
    return tuple(None if t is None else t.to(device) for t in ts)


def _grads(q, k, v, cfg, index, do, **kw):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = moba.moba_attention(q, k, v, cfg, index=index, **kw)
    out.backward(do)
    return out.detach(), q.grad, k.grad, v.grad


# ---------------------------------------------------------------------------
# golden vectors produced by the reference oracle
# ---------------------------------------------------------------------------

def test_golden_selection_output_and_gradients(golden, device, kernel_path):
    dt = golden.low_dtype
    cfg = golden.config()
    q, k, v, cu = _dev(golden.q.to(dt), golden.k.to(dt), golden.v.to(dt), golden.cu, device=device)
    index = moba.build_csc_fused(q, k, cfg, cu_seqlens=cu, max_seqlen=golden.max_seqlen)
    mask = moba.csc_to_mask(index, q.shape[1]).cpu()
    assert mask.shape == golden.mask.shape
    assert torch.equal(mask, golden.mask), "selection differs from the reference oracle"

    out = moba.moba_forward(q, k, v, cfg, index=index)
    live = ~torch.isnan(golden.out)
    assert torch.equal(torch.isnan(out.cpu().float()), ~live)
    err = max_abs_error(out.cpu().float()[live], golden.out[live])
    assert err <= ATOL[dt], f"forward error {err:.3e}"
    if golden.out_low is not None:
        ref_err = max_abs_error(golden.out_low.float()[live], golden.out[live])
        assert err <= max(TOLERANCE_FACTOR * ref_err, TOLERANCE_FLOOR)

    if golden.has_grads:
        do = golden.do.to(dt).to(device)
        _, dq, dk, dv = _grads(q, k, v, cfg, index, do)
        for name, got, want in (("dq", dq, golden.dq), ("dk", dk, golden.dk), ("dv", dv, golden.dv)):
            e = max_abs_error(got.cpu().float(), want)
            assert e <= ATOL[dt], f"{name} error {e:.3e}"


# ---------------------------------------------------------------------------
# seeded sweeps against the oracle (sizes the oracle finishes in seconds)
# ---------------------------------------------------------------------------

SWEEP = [
    # shape [B,S,Hq,D], Hkv, block, top_k, dtype
    ((1, 1024, 4, 128), 4, 32, 4, torch.bfloat16),
    ((2, 1024, 4, 128), 4, 64, 8, torch.bfloat16),
    ((1, 2048, 4, 64), 4, 128, 8, torch.bfloat16),
    ((1, 2048, 2, 128), 2, 128, 8, torch.bfloat16),
    ((1, 4096, 2, 64), 2, 128, 12, torch.bfloat16),
    ((1, 2048, 8, 128), 2, 128, 8, torch.bfloat16),     # grouped-query, G = 4
    ((1, 1000, 4, 64), 2, 128, 4, torch.bfloat16),      # short tail block, G = 2
    ((1, 1024, 2, 64), 2, 64, 4, torch.float16),
    ((1, 1024, 2, 64), 2, 128, 4, torch.float32),
    ((1, 512, 2, 32), 1, 32, 4, torch.float32),
]
SWEEP_IDS = [f"b{s[0]}s{s[1]}h{s[2]}kv{h}d{s[3]}-blk{b}-top{t}-{str(d).split('.')[-1]}"
             for s, h, b, t, d in SWEEP]


@pytest.mark.parametrize("shape,hkv,bs,top_k,dtype", SWEEP, ids=SWEEP_IDS)
def test_sweep_selection_forward_backward(shape, hkv, bs, top_k, dtype, device, kernel_path):
    cfg = moba.MoBAConfig(block_size=bs, top_k=top_k, dtype=dtype)
    q, k, v, do = make_qkv(shape, hkv, dtype=dtype, seed=11, with_do=True)
    qd, kd, vd, dod = _dev(q, k, v, do, device=device)

    index = moba.build_csc_fused(qd, kd, cfg)
    mask = moba.csc_to_mask(index, shape[1])
    want, scores = oracle_mask(q, k, cfg, return_scores=True)
    lib = _lib.load()
    prob = _lib.make_problem(shape, hkv, dtype, cfg)
    if lib.moba_b200_path_for(prob, _lib.STAGE_GATE) == _lib.PATH_PORTABLE or dtype == torch.float32:
        assert torch.equal(mask.cpu(), want), "portable gate must match the oracle exactly"
    else:
        differing, bad = near_tie_report(mask, want, scores, 8 if dtype == torch.bfloat16 else 11)
        assert bad == 0, f"{bad} selections differ from the oracle beyond a near tie"
        assert differing <= max(2, 1e-4 * mask.shape[0] * mask.shape[1] * mask.shape[2])

    # forward and backward with the engine's own routing held fixed
    kbar = moba.pool_blocks(kd, cfg)
    block_idx = moba.gate_select(qd, kbar, cfg)
    assert torch.equal(orc.block_idx_to_mask(block_idx.cpu(), want.shape[-1]), mask.cpu())
    t_out, t_lse, t_dq, t_dk, t_dv = oracle_forward(q, k, v, cfg, block_idx, dout=do)
    out, dq, dk, dv = _grads(qd, kd, vd, cfg, index, dod)
    for name, got, truth in (("out", out, t_out), ("dq", dq, t_dq), ("dk", dk, t_dk), ("dv", dv, t_dv)):
        e = max_abs_error(got, truth)
        assert e <= ATOL[dtype], f"{name} error {e:.3e} over {ATOL[dtype]:.0e}"
    # the inference entry point agrees with the training one bit for bit
    assert torch.equal(moba.moba_forward(qd, kd, vd, cfg, index=index), out)


def test_reference_relative_policy_bf16(device, kernel_path):
    """max|ours - truth| <= max(2 * max|bf16 oracle - truth|, 1e-6), routing fixed."""
    shape, bs, top_k = (1, 2048, 4, 128), 128, 8
    cfg = moba.MoBAConfig(bs, top_k)
    q, k, v = make_qkv(shape, dtype=torch.bfloat16, seed=5)
    qd, kd, vd = _dev(q, k, v, device=device)
    index = moba.build_csc_fused(qd, kd, cfg)
    mask = moba.csc_to_mask(index, shape[1]).cpu()
    truth = orc.attention_dense(q.double(), k.double(), v.double(), bs, mask, query_chunk=256)
    low = orc.attention_dense(q, k, v, bs, mask, query_chunk=256)
    ref_err = max_abs_error(low, truth)
    err = max_abs_error(moba.moba_forward(qd, kd, vd, cfg, index=index), truth)
    assert err <= max(TOLERANCE_FACTOR * ref_err, TOLERANCE_FLOOR), (err, ref_err)


# ---------------------------------------------------------------------------
# transpose against the host restatement
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("shape,hkv,bs,top_k,cu", [
    ((1, 2048, 4, 64), 2, 32, 4, None),
    ((2, 1000, 2, 64), 2, 64, 8, None),
    ((1, 212, 4, 64), 2, 16, 3, [0, 80, 128, 192, 212]),
    ((1, 16384, 2, 64), 1, 16, 4, None),                 # 1024 columns, two heads per column
])
def test_transpose_matches_host_restatement_exactly(shape, hkv, bs, top_k, cu, device):
    cfg = moba.MoBAConfig(bs, top_k)
    q, k, _ = make_qkv(shape, hkv, dtype=torch.bfloat16, seed=3)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    longest = None if cu is None else max(b - a for a, b in zip(cu[:-1], cu[1:]))
    qd, kd, cud = _dev(q, k, cu_t, device=device)
    kbar = moba.pool_blocks(kd, cfg, cu_seqlens=cud, max_seqlen=longest)
    block_idx = moba.gate_select(qd, kbar, cfg, cu_seqlens=cud, max_seqlen=longest)
    index = moba.build_csc_from_indices(block_idx, kbar.shape[2], cfg, num_kv_heads=hkv,
                                        cu_seqlens=cud, max_seqlen=longest)
    want = orc.build_csc(block_idx.cpu(), kbar.shape[2], hkv, cu_seqlens=cu_t, max_seqlen=longest)
    assert torch.equal(index.col_nnz.cpu(), want["col_nnz"])
    assert torch.equal(index.col_offsets.cpu(), want["col_offsets"])
    assert torch.equal(index.order.cpu(), want["order"])
    total = want["col_nnz"].sum(dim=-1)
    for si in range(total.shape[0]):
        for h in range(total.shape[1]):
            n = int(total[si, h])
            for name in ("row_indices", "head_indices", "slot_of_pair"):
                assert torch.equal(getattr(index, name)[si, h, :n].cpu(), want[name][si, h, :n]), name
    if cu is not None:                                   # no column crosses a sequence
        m = moba.csc_to_mask(index, shape[1]).cpu()
        for i, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
            assert not m[0, :, a:b, cfg.num_blocks(b - a):].any()


def test_pooling_matches_oracle_bitwise_including_tails(device):
    for dtype in (torch.bfloat16, torch.float32, torch.float16):
        cfg = moba.MoBAConfig(48, 2)
        _, k, _ = make_qkv((2, 200, 2, 64), dtype=dtype, seed=9)
        got = moba.pool_blocks(k.to(device), cfg).cpu()
        assert torch.equal(got, orc.pool_blocks(k, 48))
    cu = torch.tensor([0, 80, 128, 192, 212], dtype=torch.int32)
    _, k, _ = make_qkv((1, 212, 2, 64), dtype=torch.bfloat16, seed=9)
    got = moba.pool_blocks(k.to(device), moba.MoBAConfig(16, 2), cu_seqlens=cu.to(device), max_seqlen=80).cpu()
    assert torch.equal(got, orc.pool_blocks(k, 16, cu, 80))


# ---------------------------------------------------------------------------
# gate edge cases the reference tests pin
# ---------------------------------------------------------------------------

def test_gate_edge_cases(device, kernel_path):
    cases = [
        ((1, 96, 2, 64), 32, 8, {}),                               # fewer blocks than top_k
        ((1, 2048, 1, 64), 16, 64, {}),                            # top_k 64
        ((1, 8192, 1, 64), 16, 8, {}),                             # 512 blocks
        ((1, 768, 2, 64), 32, 12, {}),                             # non power-of-two capacity
        ((1, 512, 2, 64), 32, 4, {"always_select_current": False}),
        ((1, 512, 2, 64), 32, 2, {"top_k_includes_current": False}),
    ]
    for shape, bs, top_k, flags in cases:
        cfg = moba.MoBAConfig(bs, top_k, **flags)
        q, k, _ = make_qkv(shape, dtype=torch.bfloat16, seed=21)
        idx = moba.gate_select(q.to(device), moba.pool_blocks(k.to(device), cfg), cfg).cpu()
        want = orc.mask_to_block_idx(oracle_mask(q, k, cfg), cfg.slots_per_query)
        assert idx.shape == want.shape
        assert torch.equal(idx, want), (shape, bs, top_k, flags)


def test_gate_breaks_exact_ties_toward_the_lower_block(device, kernel_path):
    cfg = moba.MoBAConfig(32, 4)
    q, k, _ = make_qkv((1, 512, 2, 64), dtype=torch.bfloat16, seed=2)
    k[:, :, 0] = k[:, :32, 0].repeat(1, 16, 1)              # every block of head 0 is identical
    idx = moba.gate_select(q.to(device), moba.pool_blocks(k.to(device), cfg), cfg).cpu()
    rows = torch.arange(512)
    own = rows // 32
    late = own >= 4
    assert torch.equal(idx[0, 0, late, :3], torch.tensor([0, 1, 2], dtype=torch.int32).expand(int(late.sum()), 3))
    assert torch.equal(idx[0, 0, :, :], orc.mask_to_block_idx(oracle_mask(q, k, cfg), 4)[0, 0])


# ---------------------------------------------------------------------------
# merge in isolation (synthetic partials; reference: tests/test_moba_kernel.py:119-326)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("slots", [1, 3, 5, 8, 12])
def test_merge_matches_textbook_and_ignores_poisoned_slots(slots, device):
    g = torch.Generator().manual_seed(slots)
    b, h, s, d = 2, 3, 130, 64
    m = torch.randn(b, h, s, slots, generator=g, dtype=torch.float64) * 4
    l = torch.rand(b, h, s, slots, generator=g, dtype=torch.float64) * 50 + 1
    acc = torch.randn(b, h, s, slots, d, generator=g, dtype=torch.float64) * l[..., None]
    written = torch.rand(b, h, s, slots, generator=g) < 0.7
    written[..., 0] = True
    m = torch.where(written, m, torch.full_like(m, float("-inf")))
    mg = m.max(dim=-1, keepdim=True).values
    w = torch.where(written, torch.exp2(m - mg), torch.zeros_like(m))
    den = (w * l).sum(-1)
    want = ((w[..., None] * torch.where(written[..., None], acc, torch.zeros_like(acc))).sum(-2) / den[..., None])
    want_lse = mg.squeeze(-1) + torch.log2(den)
    poison = torch.where(written[..., None], acc, torch.full_like(acc, float("nan")))
    lp = torch.where(written, l, torch.full_like(l, float("nan")))
    out, lse = moba.combine_partials(m.float().to(device), lp.float().to(device), poison.float().to(device),
                                     torch.float32, return_lse=True)
    assert out.shape == (b, s, h, d)
    assert max_abs_error(out.permute(0, 2, 1, 3), want) < 1e-5
    assert max_abs_error(lse, want_lse) < 1e-5
    # native entry: dominant slot and shift invariance
    shifted, _ = moba.combine_partials((m + 40).float().to(device), lp.float().to(device),
                                       poison.float().to(device), torch.float32, return_lse=True)
    assert max_abs_error(shifted, out) < 1e-5


# ---------------------------------------------------------------------------
# invariants that need no oracle (reference: tests/test_kernel_invariants.py)
# ---------------------------------------------------------------------------

def test_determinism_causality_and_block_perturbation(device, kernel_path):
    cfg = moba.MoBAConfig(128, 4)
    shape = (1, 2048, 2, 64)
    q, k, v, do = _dev(*make_qkv(shape, dtype=torch.bfloat16, seed=8, with_do=True), device=device)
    index = moba.build_csc_fused(q, k, cfg)
    a = _grads(q, k, v, cfg, index, do)
    b = _grads(q, k, v, cfg, index, do)
    for x, y in zip(a, b):
        assert torch.equal(x, y), "repeated runs differ"
    # dispatch order is irrelevant (doubles as a write-race detector): the portable kernels walk
    # `order`, the tensor-core kernels the work items
    flipped = dataclasses.replace(index, order=index.order.flip(-1).contiguous(),
                                  work_items=index.work_items.flip(2).contiguous())
    for x, y in zip(a, _grads(q, k, v, cfg, flipped, do)):
        assert torch.equal(x, y), "results depend on the dispatch order"
    # perturbing one block's values changes exactly the queries that selected it
    mask = moba.csc_to_mask(index, shape[1])
    v2 = v.clone()
    v2[:, 3 * 128:4 * 128, 1] += 1.0
    o2 = moba.moba_forward(q, k, v2, cfg, index=index)
    changed = (o2 != a[0]).any(dim=-1)                       # [B,S,H]
    assert torch.equal(changed[0, :, 1], mask[0, 1, :, 3])
    assert not changed[0, :, 0].any()
    # causality: changing the future never changes the past
    q3, k3, v3 = q.clone(), k.clone(), v.clone()
    for t in (q3, k3, v3):
        t[:, 1500:] = 0.5
    o3 = moba.moba_forward(q3, k3, v3, cfg)
    assert torch.equal(o3[:, :1500], moba.moba_forward(q, k, v, cfg)[:, :1500])


def test_unselected_blocks_get_exact_zero_gradients(device, kernel_path):
    cfg = moba.MoBAConfig(64, 4, always_select_current=False)
    shape = (1, 1024, 2, 64)
    q, k, v, do = _dev(*make_qkv(shape, dtype=torch.bfloat16, seed=4, with_do=True), device=device)
    index = moba.build_csc_fused(q, k, cfg)
    empty = (index.col_nnz == 0).nonzero().tolist()
    assert empty, "no unselected block, nothing is being checked"
    dk0 = torch.full_like(k, 7.0)                             # stale values must be overwritten
    del dk0
    _, _, dk, dv = _grads(q, k, v, cfg, index, do)
    for _, h, blk in empty:
        assert not dk[0, blk * 64:(blk + 1) * 64, h].any()
        assert not dv[0, blk * 64:(blk + 1) * 64, h].any()


def test_kv_heads_per_pass_is_bitwise_the_whole_op(device, kernel_path):
    """Running the op a few KV heads at a time (host-side chunking that bounds the partial
    buffers) gives the same bits as one call: KV heads are independent."""
    cfg = moba.MoBAConfig(block_size=128, top_k=4, dtype=torch.bfloat16)
    q, k, v, do = make_qkv((1, 1024, 12, 64), 3, dtype=torch.bfloat16, seed=23, with_do=True)
    qd, kd, vd, dod = _dev(q, k, v, do, device=device)

    def run(**kw):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (qd, kd, vd))
        out = moba.moba_attention(qq, kk, vv, cfg, **kw)
        out.backward(dod)
        return out.detach(), qq.grad, kk.grad, vv.grad

    whole = run()
    for per_pass in (1, 2):                                  # 2: the last pass holds one head
        for got, want in zip(run(kv_heads_per_pass=per_pass), whole):
            assert torch.equal(got, want)
        assert torch.equal(moba.moba_forward(qd, kd, vd, cfg, kv_heads_per_pass=per_pass), whole[0])
    assert torch.equal(moba.moba_forward(qd, kd, vd, cfg, kv_heads_per_pass=8), whole[0])


def test_gqa_equals_expanded_kv(device, kernel_path):
    cfg = moba.MoBAConfig(64, 4)
    q, k, v, do = make_qkv((1, 1024, 8, 64), 2, dtype=torch.bfloat16, seed=6, with_do=True)
    qd, kd, vd, dod = _dev(q, k, v, do, device=device)
    ke, ve = kd.repeat_interleave(4, dim=2), vd.repeat_interleave(4, dim=2)
    shared = _grads(qd, kd, vd, cfg, None, dod)
    expanded = _grads(qd, ke, ve, cfg, None, dod)
    assert torch.equal(moba.csc_to_mask(moba.build_csc_fused(qd, kd, cfg), 1024),
                       moba.csc_to_mask(moba.build_csc_fused(qd, ke, cfg), 1024))
    assert torch.equal(shared[0], expanded[0]) and torch.equal(shared[1], expanded[1])
    for got, exp in ((shared[2], expanded[2]), (shared[3], expanded[3])):
        folded = exp.float().view(1, 1024, 2, 4, 64).sum(3)
        assert torch.allclose(got.float(), folded, rtol=3e-2, atol=2e-3)


def test_packed_equals_per_sequence_bitwise_forward(device, kernel_path):
    cu = [0, 300, 428, 1000, 1024]
    cfg = moba.MoBAConfig(64, 3)
    q, k, v, do = make_qkv((1, 1024, 4, 64), 2, dtype=torch.bfloat16, seed=13, with_do=True)
    qd, kd, vd, dod = _dev(q, k, v, do, device=device)
    cud = torch.tensor(cu, dtype=torch.int32, device=device)
    out, dq, dk, dv = _grads(qd, kd, vd, cfg, None, dod, cu_seqlens=cud, max_seqlen=572)
    for a, b in zip(cu[:-1], cu[1:]):
        o1, q1, k1, v1 = _grads(qd[:, a:b], kd[:, a:b], vd[:, a:b], cfg, None, dod[:, a:b])
        assert torch.equal(out[:, a:b], o1), "packed forward differs from the sequence run alone"
        assert torch.equal(dq[:, a:b], q1)
        assert torch.allclose(dk[:, a:b].float(), k1.float(), rtol=2e-2, atol=1e-3)
        assert torch.allclose(dv[:, a:b].float(), v1.float(), rtol=2e-2, atol=1e-3)
    # and against the oracle with per-sequence blocks
    mask = moba.csc_to_mask(moba.build_csc_fused(qd, kd, cfg, cu_seqlens=cud, max_seqlen=572), 1024).cpu()
    assert torch.equal(mask, oracle_mask(q, k, cfg, cu=torch.tensor(cu, dtype=torch.int32), max_seqlen=572))


def test_non_causal_own_block(device, kernel_path):
    cfg = moba.MoBAConfig(64, 3)
    q, k, v = make_qkv((1, 512, 2, 64), dtype=torch.bfloat16, seed=17)
    qd, kd, vd = _dev(q, k, v, device=device)
    kbar = moba.pool_blocks(kd, cfg)
    block_idx = moba.gate_select(qd, kbar, cfg)
    out = moba.moba_forward(qd, kd, vd, cfg, causal=False)
    truth, _ = oracle_forward(q, k, v, cfg, block_idx, causal=False)
    assert max_abs_error(out, truth) <= ATOL[torch.bfloat16]


@pytest.mark.parametrize("d,s", [(64, 1024), (128, 2048)], ids=["d64", "d128"])
def test_float32_partials_option(d, s, device, kernel_path):
    """float32 partial outputs leave the forward kernel by another route than 16-bit ones
    (straight from registers, not through the staging tile and, at head_dim 128, not through
    the mover warps): both must give the merged output of the oracle."""
    cfg = moba.MoBAConfig(128, 4)
    q, k, v = make_qkv((1, s, 4, d), dtype=torch.bfloat16, seed=19, hkv=2)
    qd, kd, vd = _dev(q, k, v, device=device)
    a = moba.moba_forward(qd, kd, vd, cfg)
    b = moba.moba_forward(qd, kd, vd, cfg, partials_dtype=torch.float32)
    assert max_abs_error(a, b) <= 2e-2
    block_idx = moba.gate_select(qd, moba.pool_blocks(kd, cfg), cfg)
    truth, _ = oracle_forward(q, k, v, cfg, block_idx)
    assert max_abs_error(b, truth) <= ATOL[torch.bfloat16]


def test_no_host_synchronisation_on_the_hot_path(device):
    cfg = moba.MoBAConfig(128, 8)
    q, k, v, do = _dev(*make_qkv((1, 2048, 2, 64), dtype=torch.bfloat16, seed=1, with_do=True), device=device)
    q.requires_grad_(True)
    moba.moba_attention(q, k, v, cfg).backward(do)          # warm: allocator, library load
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        moba.moba_attention(q, k, v, cfg).backward(do)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()


def test_backend_adapter_runs_the_engine(device):
    from moba_triton_b200.adapter import B200Backend
    b = B200Backend()
    cfg = moba.MoBAConfig(128, 4)
    assert b.is_available(cfg) == (True, "")
    q, k, v = _dev(*make_qkv((1, 1024, 2, 64), dtype=torch.bfloat16, seed=3), device=device)
    out = b.forward(q, k, v, cfg)
    assert torch.equal(out, moba.moba_forward(q, k, v, cfg))
    assert torch.equal(b.forward_grad(q, k, v, cfg), out)
    assert torch.equal(b.selection(q, k, cfg).cpu(), oracle_mask(q.cpu(), k.cpu(), cfg))


def test_query_chunking_gives_the_whole_op(device, kernel_path):
    """Running the op a window of query rows at a time (host-side chunking along the query
    axis, which bounds the partial buffers whatever the number of heads): every (query,
    block) pair is computed as in the whole call, so O and dQ are the same bits; dK/dV are
    sums over the windows."""
    cfg = moba.MoBAConfig(block_size=128, top_k=4, dtype=torch.bfloat16)
    q, k, v, do = make_qkv((2, 1536, 4, 64), 2, dtype=torch.bfloat16, seed=29, with_do=True)
    qd, kd, vd, dod = _dev(q, k, v, do, device=device)

    def run(**kw):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (qd, kd, vd))
        out = moba.moba_attention(qq, kk, vv, cfg, **kw)
        out.backward(dod)
        return out.detach(), qq.grad, kk.grad, vv.grad

    whole = run()
    for chunk in (512, 640, 100, 4096):                     # aligned, ragged, below a block, above S
        got = run(query_chunk=chunk)
        assert torch.equal(got[0], whole[0]), f"output differs at query_chunk {chunk}"
        assert torch.equal(got[1], whole[1]), f"dQ differs at query_chunk {chunk}"
        assert torch.allclose(got[2].float(), whole[2].float(), rtol=2e-2, atol=2e-3)
        assert torch.allclose(got[3].float(), whole[3].float(), rtol=2e-2, atol=2e-3)
        assert torch.equal(moba.moba_forward(qd, kd, vd, cfg, query_chunk=chunk), whole[0])
    with pytest.raises(ValueError, match="query_chunk"):
        moba.moba_forward(qd, kd, vd, cfg, query_chunk=512, kv_heads_per_pass=1)
    # the partial buffers of a chunked call hold one window
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats(device)
    base = torch.cuda.memory_allocated(device)
    moba.moba_forward(qd, kd, vd, cfg, query_chunk=256)
    torch.cuda.synchronize()
    chunked_peak = torch.cuda.max_memory_allocated(device) - base
    torch.cuda.reset_peak_memory_stats(device)
    moba.moba_forward(qd, kd, vd, cfg)
    torch.cuda.synchronize()
    whole_peak = torch.cuda.max_memory_allocated(device) - base
    assert chunked_peak < 0.6 * whole_peak, (chunked_peak, whole_peak)


def test_candidate_window_gate_on_both_kernel_families(device, kernel_path):
    cfg = moba.MoBAConfig(32, 4, gate_window=5, gate_sinks=2)
    q, k, _ = make_qkv((2, 1024, 2, 64), dtype=torch.bfloat16, seed=33)
    idx = moba.gate_select(q.to(device), moba.pool_blocks(k.to(device), cfg), cfg).cpu()
    want = orc.mask_to_block_idx(oracle_mask(q, k, cfg), cfg.slots_per_query)
    assert torch.equal(idx, want)
    wide = moba.MoBAConfig(32, 4, gate_window=64)
    idx2 = moba.gate_select(q.to(device), moba.pool_blocks(k.to(device), wide), wide).cpu()
    assert torch.equal(idx2, orc.mask_to_block_idx(oracle_mask(q, k, moba.MoBAConfig(32, 4)), 4))
