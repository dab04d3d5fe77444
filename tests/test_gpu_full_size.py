"""Checks at the benchmark's full size ([1,131072,4,64] bf16, block 128, top_k 8),
where the oracle cannot be run over everything: closed-form pair counts,
structural invariants of the routing, exact linearity of the backward, and the
oracle on a seeded sample of queries and of key/value blocks."""

import pytest
import torch

import moba_triton_b200 as moba
from oracle import moba_oracle as orc

from conftest import make_qkv
from helpers import max_abs_error

pytestmark = pytest.mark.gpu

S, H, D, BS, TOPK = 131072, 4, 64, 128, 8


@pytest.fixture(scope="module")
def full(device):
    cfg = moba.MoBAConfig(BS, TOPK)
    q, k, v, do = make_qkv((1, S, H, D), dtype=torch.bfloat16, seed=0, with_do=True)
    qd, kd, vd, dod = (t.to(device) for t in (q, k, v, do))
    kbar = moba.pool_blocks(kd, cfg)
    block_idx = moba.gate_select(qd, kbar, cfg)
    index = moba.build_csc_from_indices(block_idx, kbar.shape[2], cfg, num_kv_heads=H)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (qd, kd, vd))
    out = moba.moba_attention(qg, kg, vg, cfg, index=index)
    out.backward(dod)
    torch.cuda.synchronize()
    return dict(cfg=cfg, q=q, k=k, v=v, do=do, qd=qd, kd=kd, vd=vd, dod=dod, kbar=kbar,
                block_idx=block_idx, index=index, out=out.detach(), dq=qg.grad, dk=kg.grad, dv=vg.grad)


def test_routing_structure_and_pair_counts(full):
    idx = full["block_idx"]                                     # [1,H,S,8]
    own = (torch.arange(S, device=idx.device) // BS).view(1, 1, S)
    valid = idx >= 0
    count = valid.sum(-1)
    assert torch.equal(count, torch.clamp(own + 1, max=TOPK).expand_as(count))
    last = idx.gather(-1, (count - 1).unsqueeze(-1)).squeeze(-1)
    assert torch.equal(last, own.expand_as(last)), "the own block must be the highest selected id"
    nxt = torch.where(valid[..., 1:], idx[..., 1:], torch.full_like(idx[..., 1:], 1 << 30))
    assert bool((idx[..., :-1] < nxt).all()), "ids must ascend, padding last"
    pairs = int(valid.sum())
    assert pairs == H * orc.selected_pairs(S, BS, TOPK) == 4179968
    ix = full["index"]
    assert int(ix.col_nnz.sum()) == pairs
    assert torch.equal(ix.col_offsets[..., 1:], ix.col_nnz.cumsum(-1).to(torch.int32))
    assert torch.equal(ix.col_nnz.gather(-1, ix.order.long()).sort(-1, descending=True).values,
                       ix.col_nnz.gather(-1, ix.order.long()))
    # every column lists exactly the queries whose block_idx names it (checked on three columns)
    for h, blk in ((0, 0), (1, 517), (3, 1023)):
        lo, n = int(ix.col_offsets[0, h, blk]), int(ix.col_nnz[0, h, blk])
        rows = ix.row_indices[0, h, lo:lo + n].long()
        assert bool((ix.head_indices[0, h, lo:lo + n] == h).all())
        want = (idx[0, h] == blk).any(-1).nonzero().squeeze(-1)
        assert torch.equal(rows, want)


def test_selection_matches_oracle_on_sampled_queries(full):
    g = torch.Generator().manual_seed(5)
    rows = torch.randint(BS, S, (768,), generator=g)
    kbar = orc.pool_blocks(full["k"], BS)                       # [1,H,nb,D] on the host
    assert torch.equal(full["kbar"].cpu(), kbar), "block means must match the oracle bit for bit"
    differing = 0
    for h in range(H):
        sc = orc.gate_scores(full["q"][0, rows][:, h:h + 1], kbar[0, h:h + 1])[0].double()   # [n, nb]
        own = rows // BS
        for i in range(rows.numel()):
            s = sc[i, :own[i]]
            order = torch.argsort(s, descending=True, stable=True)[:TOPK - 1]
            want = set(order.tolist()) | {int(own[i])}
            got = set(x for x in full["block_idx"][0, h, rows[i]].tolist() if x >= 0)
            if got != want:
                differing += 1
                a, b = sorted(got - want), sorted(want - got)
                assert len(a) == len(b) == 1, (got, want)
                step = 2.0 ** -7 * max(abs(float(s[a[0]])), abs(float(s[b[0]])))
                assert abs(float(s[a[0]]) - float(s[b[0]])) <= step, "differs beyond a near tie"
    assert differing <= 2


def _oracle_rows(full, h, rows):
    """float64 attention for the sampled queries of head h: (out, lse2, p, keys index)."""
    q, k, v = full["q"][0, :, h].double(), full["k"][0, :, h].double(), full["v"][0, :, h].double()
    idx = full["block_idx"][0, h].cpu()[rows].long()            # [n, 8]
    kp = idx.clamp(min=0).unsqueeze(-1) * BS + torch.arange(BS)  # [n, 8, 128]
    ok = (idx >= 0).unsqueeze(-1) & (kp <= rows.view(-1, 1, 1))
    logits = torch.einsum("nd,nkjd->nkj", q[rows], k[kp]) * D ** -0.5
    logits = logits.masked_fill(~ok, float("-inf")).flatten(1)
    lse = torch.logsumexp(logits, dim=-1)
    p = torch.exp(logits - lse[:, None])
    out = torch.einsum("nj,njd->nd", p, v[kp.flatten(1)])
    return out, lse * orc.LOG2E, p, kp.flatten(1)


def test_forward_and_dq_match_oracle_on_sampled_queries(full):
    g = torch.Generator().manual_seed(6)
    rows = torch.randint(0, S, (512,), generator=g)
    for h in (0, 3):
        out, _, p, kidx = _oracle_rows(full, h, rows)
        assert max_abs_error(full["out"][0, rows, h], out) <= 2e-2
        do = full["do"][0, rows, h].double()
        k, v = full["k"][0, :, h].double(), full["v"][0, :, h].double()
        dp = torch.einsum("nd,njd->nj", do, v[kidx])
        ds = p * (dp - (p * dp).sum(-1, keepdim=True)) * D ** -0.5
        dq = torch.einsum("nj,njd->nd", ds, k[kidx])
        assert max_abs_error(full["dq"][0, rows, h], dq) <= 2e-2


def test_dk_dv_match_oracle_on_sampled_blocks(full):
    ix = full["index"]
    for h, blk in ((0, 3), (2, 600), (1, 1023)):
        lo, n = int(ix.col_offsets[0, h, blk]), int(ix.col_nnz[0, h, blk])
        rows = ix.row_indices[0, h, lo:lo + n].cpu().long()
        _, _, p, kidx = _oracle_rows(full, h, rows)
        do = full["do"][0, rows, h].double()
        q, v = full["q"][0, rows, h].double(), full["v"][0, :, h].double()
        dp = torch.einsum("nd,njd->nj", do, v[kidx])
        ds = p * (dp - (p * dp).sum(-1, keepdim=True)) * D ** -0.5
        mine = (kidx >= blk * BS) & (kidx < (blk + 1) * BS)       # entries of this block per query
        pos = (kidx - blk * BS).clamp(0, BS - 1)
        dv = torch.zeros(BS, D, dtype=torch.float64)
        dk = torch.zeros(BS, D, dtype=torch.float64)
        w_p = torch.where(mine, p, torch.zeros_like(p))
        w_s = torch.where(mine, ds, torch.zeros_like(ds))
        dv.index_add_(0, pos.flatten(), (w_p.unsqueeze(-1) * do.unsqueeze(1)).flatten(0, 1))
        dk.index_add_(0, pos.flatten(), (w_s.unsqueeze(-1) * q.unsqueeze(1)).flatten(0, 1))
        sl = slice(blk * BS, (blk + 1) * BS)
        scale = max(1.0, float(dv.abs().max()), float(dk.abs().max()))
        assert max_abs_error(full["dv"][0, sl, h], dv) <= 2e-2 * scale
        assert max_abs_error(full["dk"][0, sl, h], dk) <= 2e-2 * scale


def test_backward_is_exactly_linear_in_the_upstream_gradient(full):
    cfg = full["cfg"]
    q, k, v = (full[n].clone().requires_grad_(True) for n in ("qd", "kd", "vd"))
    moba.moba_attention(q, k, v, cfg, index=full["index"]).backward(full["dod"] * 2)   # power of two: exact
    torch.cuda.synchronize()
    assert torch.equal(q.grad, full["dq"] * 2)
    assert torch.equal(k.grad, full["dk"] * 2)
    assert torch.equal(v.grad, full["dv"] * 2)


def test_outputs_are_convex_combinations_of_values(full):
    vmax = full["vd"].float().abs().amax(dim=1, keepdim=True)    # per head and channel
    assert bool((full["out"].float().abs() <= vmax * 1.01 + 1e-3).all())
    assert not bool(torch.isnan(full["out"].float()).any())
