"""CPU oracle for the MoBA attention path.  TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product package never does.

It restates, in plain PyTorch on the host, the algorithm the reference defines
in `src/moba/naive.py` (pool :23-61, gate :64-146, packed selection :149-189,
attention :206-329), in two forms:

* a *dense* form that materialises the [S, S] logits like the reference does
  (small sequences, the definition), and
* a *sparse* form that gathers only the selected key blocks per query and has
  closed-form gradients (long sequences, and the timed CPU baseline).

Parity pin: `tests/golden/` holds outputs of the reference's own
`moba.naive` functions (selection masks, outputs, autograd gradients) that
`tests/test_oracle_golden.py` replays against both forms.

Numerics contract of the gate (shared with the CUDA kernels so that selection
can be compared exactly, independent of summation order):

* block sum  = round_to_input_dtype( float32( exact sum ) )  -- the exact sum is
  taken in float64, where <= 2^16 low-precision addends cannot round;
* block mean = round_to_input_dtype( float32(sum) / float32(occupancy) );
* score      = round_to_input_dtype( float32( exact dot(q, mean) ) ), unscaled;
* candidates are blocks strictly before the query's own block; rank by score
  descending, ties to the lower block id; the own block is added, never ranked.

The reference accumulates the same quantities in float32 (pooling.py:77-95,
gating.py:231-237), which differs from the exact value only when a float32
partial sum rounds across a low-precision rounding boundary.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------
# configuration helpers (plain ints so this file needs nothing from the product)
# --------------------------------------------------------------------------

def num_blocks(seq_len: int, block_size: int) -> int:
    return -(-seq_len // block_size)


def past_budget(top_k: int, nb: int, always_current: bool = True,
                includes_current: bool = True) -> int:
    """reference: src/moba/config.py:69-84"""
    take = top_k - (1 if (always_current and includes_current) else 0)
    return max(0, min(take, nb))


def _spans(total: int, cu_seqlens) -> list[tuple[int, int]]:
    if cu_seqlens is None:
        return [(0, total)]
    b = [int(x) for x in (cu_seqlens.tolist() if hasattr(cu_seqlens, "tolist") else cu_seqlens)]
    return list(zip(b[:-1], b[1:]))


def _round_like(x64: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """float64 -> float32 -> dtype, the two-step rounding the kernels use."""
    if dtype == torch.float64:
        return x64
    return x64.to(torch.float32).to(dtype)


# --------------------------------------------------------------------------
# gate: pool, score, select
# --------------------------------------------------------------------------

def pool_blocks(k: torch.Tensor, block_size: int, cu_seqlens=None,
                max_seqlen: Optional[int] = None) -> torch.Tensor:
    """Mean key of every block (reference: naive.py:23-61, pooling.py:25-95).

    k: [B, S, Hkv, D] or packed [1, T, Hkv, D].
    Returns [B, Hkv, nb, D], or [n_seq, Hkv, cdiv(max_seqlen, bs), D] when
    packed (rows of short sequences are zero past their own block count).
    """
    dt = k.dtype
    if cu_seqlens is None:
        pieces = [k[b] for b in range(k.shape[0])]
        nb_out = num_blocks(k.shape[1], block_size)
    else:
        spans = _spans(k.shape[1], cu_seqlens)
        pieces = [k[0, lo:hi] for lo, hi in spans]
        longest = max(hi - lo for lo, hi in spans) if max_seqlen is None else max_seqlen
        nb_out = num_blocks(longest, block_size)
    h, d = k.shape[2], k.shape[3]
    out = torch.zeros(len(pieces), h, nb_out, d, dtype=dt)
    for i, piece in enumerate(pieces):
        s = piece.shape[0]
        nb = num_blocks(s, block_size)
        pad = nb * block_size - s
        p64 = torch.nn.functional.pad(piece.to(torch.float64), (0, 0, 0, 0, 0, pad))
        sums = p64.view(nb, block_size, h, d).sum(dim=1)          # exact
        sums = _round_like(sums, dt)                               # round #1
        occ = torch.full((nb,), float(block_size), dtype=torch.float32)
        occ[-1] = block_size - pad
        if dt == torch.float64:
            mean = sums / occ.to(torch.float64).view(nb, 1, 1)
        else:
            mean = (sums.to(torch.float32) / occ.view(nb, 1, 1)).to(dt)   # round #2
        out[i, :, :nb] = mean.permute(1, 0, 2)
    return out


def gate_scores(q_seq: torch.Tensor, kbar_seq: torch.Tensor) -> torch.Tensor:
    """q_seq [S, Hq, D], kbar_seq [Hkv, nb, D] -> scores [Hq, S, nb] in q dtype
    (unscaled; reference: naive.py:104-109, gating.py:231-237)."""
    hq, hkv = q_seq.shape[1], kbar_seq.shape[0]
    g = hq // hkv
    kb = kbar_seq.to(torch.float64).repeat_interleave(g, dim=0)   # head h -> h // g
    s64 = torch.einsum("shd,hnd->hsn", q_seq.to(torch.float64), kb)
    return _round_like(s64, q_seq.dtype)


def select_blocks_seq(scores: torch.Tensor, block_size: int, top_k: int,
                      always_current: bool = True,
                      includes_current: bool = True,
                      gate_window: Optional[int] = None, gate_sinks: int = 0) -> torch.Tensor:
    """scores [Hq, S, nb] -> bool mask [Hq, S, nb] (reference: naive.py:111-146).

    `gate_window` / `gate_sinks` are this engine's candidate restriction (no counterpart in
    the reference): only the `gate_window` blocks before the own block and the first
    `gate_sinks` blocks are ranked."""
    hq, s, nb = scores.shape
    own = torch.arange(s) // block_size
    blocks = torch.arange(nb)
    is_past = blocks.view(1, nb) < own.view(s, 1)
    if gate_window is not None:
        is_past &= (blocks.view(1, nb) < gate_sinks) | (blocks.view(1, nb) >= own.view(s, 1) - gate_window)
    masked = scores.to(torch.float64).masked_fill(~is_past.view(1, s, nb), float("-inf"))
    order = torch.argsort(masked, dim=-1, descending=True, stable=True)
    take = past_budget(top_k, nb, always_current, includes_current)
    sel = torch.zeros(hq, s, nb, dtype=torch.bool)
    sel.scatter_(-1, order[..., :take], True)
    sel &= is_past.view(1, s, nb)
    if always_current:
        sel |= (blocks.view(1, nb) == own.view(s, 1)).view(1, s, nb)
    return sel


def selection_mask(q: torch.Tensor, k: torch.Tensor, block_size: int, top_k: int,
                   cu_seqlens=None, max_seqlen: Optional[int] = None,
                   always_current: bool = True, includes_current: bool = True,
                   return_scores: bool = False, gate_window: Optional[int] = None, gate_sinks: int = 0):
    """Bool [B|1, Hq, S|T, nb]; packed block ids are sequence-local and the last
    axis is sized by the longest sequence (reference: naive.py:149-189)."""
    kbar = pool_blocks(k, block_size, cu_seqlens, max_seqlen)
    nbw = kbar.shape[2]
    bq, t, hq, _ = q.shape
    out = torch.zeros(bq, hq, t, nbw, dtype=torch.bool)
    sc_out = torch.full((bq, hq, t, nbw), float("-inf"), dtype=torch.float64) if return_scores else None
    if cu_seqlens is None:
        items = [(b, 0, t, b) for b in range(bq)]
    else:
        items = [(0, lo, hi, i) for i, (lo, hi) in enumerate(_spans(t, cu_seqlens))]
    for b, lo, hi, row in items:
        nb = num_blocks(hi - lo, block_size)
        sc = gate_scores(q[b, lo:hi], kbar[row, :, :nb])
        out[b, :, lo:hi, :nb] = select_blocks_seq(sc, block_size, top_k,
                                                  always_current, includes_current, gate_window, gate_sinks)
        if return_scores:
            sc_out[b, :, lo:hi, :nb] = sc.to(torch.float64)
    return (out, sc_out) if return_scores else out


def mask_to_block_idx(mask: torch.Tensor, slots: int) -> torch.Tensor:
    """Bool [B,H,S,nb] -> int32 [B,H,S,slots], ascending ids, -1 padded
    (the layout reference gating.py:365-369 emits)."""
    b, h, s, nb = mask.shape
    ids = torch.arange(nb, dtype=torch.int64).expand(b, h, s, nb)
    key = torch.where(mask, ids, torch.full_like(ids, nb))
    ordered = key.sort(dim=-1).values[..., :slots]
    if ordered.shape[-1] < slots:
        ordered = torch.nn.functional.pad(ordered, (0, slots - ordered.shape[-1]), value=nb)
    return torch.where(ordered < nb, ordered, torch.full_like(ordered, -1)).to(torch.int32)


def block_idx_to_mask(block_idx: torch.Tensor, nb: int) -> torch.Tensor:
    b, h, s, kk = block_idx.shape
    mask = torch.zeros(b, h, s, nb + 1, dtype=torch.bool)
    idx = torch.where(block_idx >= 0, block_idx.to(torch.int64), torch.full_like(block_idx, nb, dtype=torch.int64))
    mask.scatter_(-1, idx, True)
    return mask[..., :nb]


# --------------------------------------------------------------------------
# attention, dense form (the definition; reference: naive.py:206-329)
# --------------------------------------------------------------------------

def attention_dense(q, k, v, block_size: int, selected: torch.Tensor,
                    cu_seqlens=None, query_chunk: Optional[int] = None):
    """Masked dense attention in the dtype of q. selected: [B|1,Hq,S|T,nb] bool."""
    if cu_seqlens is not None:
        out = torch.empty_like(q)
        for lo, hi in _spans(q.shape[1], cu_seqlens):
            nb = num_blocks(hi - lo, block_size)
            out[:, lo:hi] = attention_dense(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi],
                                            block_size, selected[:, :, lo:hi, :nb],
                                            query_chunk=query_chunk)
        return out
    b, s, hq, d = q.shape
    g = hq // k.shape[2]
    kx = k.repeat_interleave(g, dim=2) if g > 1 else k
    vx = v.repeat_interleave(g, dim=2) if g > 1 else v
    pos = torch.arange(s)
    blk = pos // block_size
    step = s if query_chunk is None else min(query_chunk, s)
    out = torch.empty_like(q)
    for lo in range(0, s, step):
        hi = min(lo + step, s)
        vis = selected[:, :, lo:hi][..., blk] & (pos[lo:hi].view(-1, 1) >= pos.view(1, -1))
        logits = torch.einsum("bihd,bjhd->bhij", q[:, lo:hi], kx) * d ** -0.5
        probs = torch.softmax(logits.masked_fill(~vis, float("-inf")), dim=-1)
        out[:, lo:hi] = torch.einsum("bhij,bjhd->bihd", probs, vx)
    return out


# --------------------------------------------------------------------------
# attention, sparse form with closed-form gradients
# --------------------------------------------------------------------------

def _blocked(x_seq: torch.Tensor, block_size: int, nb: int) -> torch.Tensor:
    """[S, H, D] -> [H, nb, bs, D], zero padded."""
    s, h, d = x_seq.shape
    pad = nb * block_size - s
    xp = torch.nn.functional.pad(x_seq, (0, 0, 0, 0, 0, pad))
    return xp.view(nb, block_size, h, d).permute(2, 0, 1, 3)


def attention_sparse(q, k, v, block_size: int, block_idx: torch.Tensor,
                     cu_seqlens=None, causal: bool = True, dout=None,
                     compute_dtype=torch.float32, row_chunk: int = 1024):
    """Gathers each query's selected blocks; exact softmax over them.

    q [B,S,Hq,D], k/v [B,S,Hkv,D] (or packed with cu_seqlens);
    block_idx int32 [B|1, Hq, S|T, slots], sequence-local ids, -1 padded.
    Returns (out [like q, compute dtype], lse [B|1,Hq,S|T] in log2 units) and,
    when `dout` is given, also (dq, dk, dv) in the compute dtype.

    `causal=False` removes only the mask inside the query's own block, as the
    reference kernels do (moba_fwd.py:383-388).
    """
    cd = compute_dtype
    bq, t, hq, d = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    scale = d ** -0.5
    out = torch.zeros(bq, t, hq, d, dtype=cd)
    lse = torch.full((bq, hq, t), float("-inf"), dtype=cd)
    want_grad = dout is not None
    if want_grad:
        dq = torch.zeros(bq, t, hq, d, dtype=cd)
        dk = torch.zeros(bq, t, hkv, d, dtype=cd)
        dv = torch.zeros(bq, t, hkv, d, dtype=cd)
    if cu_seqlens is None:
        items = [(b, 0, t) for b in range(bq)]
    else:
        items = [(0, lo, hi) for lo, hi in _spans(t, cu_seqlens)]
    for b, lo, hi in items:
        s = hi - lo
        nb = num_blocks(s, block_size)
        kb = _blocked(k[b, lo:hi].to(cd), block_size, nb)      # [Hkv, nb, bs, D]
        vb = _blocked(v[b, lo:hi].to(cd), block_size, nb)
        if want_grad:
            dkb = torch.zeros_like(kb)
            dvb = torch.zeros_like(vb)
        key_pos = (torch.arange(nb).view(nb, 1) * block_size
                   + torch.arange(block_size).view(1, block_size))     # [nb, bs]
        for h in range(hq):
            hk = h // g
            for r0 in range(0, s, row_chunk):
                r1 = min(r0 + row_chunk, s)
                idx = block_idx[b, h, lo + r0:lo + r1].to(torch.int64)    # [R, K]
                valid = idx >= 0
                safe = idx.clamp(min=0)
                kg = kb[hk][safe]                                          # [R, K, bs, D]
                vg = vb[hk][safe]
                qr = q[b, lo + r0:lo + r1, h].to(cd)                       # [R, D]
                logits = torch.einsum("rd,rkjd->rkj", qr, kg) * scale
                kp = key_pos[safe]                                         # [R, K, bs]
                rows = torch.arange(r0, r1).view(-1, 1, 1)
                ok = valid.unsqueeze(-1) & (kp < s)
                if causal:
                    ok = ok & (kp <= rows)
                else:
                    ok = ok & (kp < (rows // block_size + 1) * block_size)
                logits = logits.masked_fill(~ok, float("-inf"))
                flat = logits.reshape(r1 - r0, -1)
                mx = flat.max(dim=-1, keepdim=True).values
                mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
                ex = torch.exp(flat - mx)
                den = ex.sum(dim=-1, keepdim=True)
                p = (ex / den).view_as(logits)                             # NaN when den == 0
                out[b, lo + r0:lo + r1, h] = torch.einsum("rkj,rkjd->rd", p, vg)
                lse[b, h, lo + r0:lo + r1] = ((mx + torch.log(den)) * LOG2E).squeeze(-1)
                if want_grad:
                    go = dout[b, lo + r0:lo + r1, h].to(cd)
                    dp = torch.einsum("rd,rkjd->rkj", go, vg)
                    p0 = torch.nan_to_num(p, nan=0.0)
                    delta = (p0 * dp).sum(dim=(1, 2), keepdim=True)
                    ds = p0 * (dp - delta) * scale
                    dq[b, lo + r0:lo + r1, h] = torch.einsum("rkj,rkjd->rd", ds, kg)
                    flat_idx = safe.reshape(-1)
                    dkb[hk].index_add_(0, flat_idx,
                                       torch.einsum("rkj,rd->rkjd", ds, qr).reshape(-1, block_size, d))
                    dvb[hk].index_add_(0, flat_idx,
                                       torch.einsum("rkj,rd->rkjd", p0, go).reshape(-1, block_size, d))
        if want_grad:
            dk[b, lo:hi] = dkb.permute(1, 2, 0, 3).reshape(nb * block_size, hkv, d)[:s]
            dv[b, lo:hi] = dvb.permute(1, 2, 0, 3).reshape(nb * block_size, hkv, d)[:s]
    if want_grad:
        return out, lse, dq, dk, dv
    return out, lse


# --------------------------------------------------------------------------
# CSR -> CSC transpose, host restatement (reference: routing.py:467-561)
# --------------------------------------------------------------------------

def build_csc(block_idx: torch.Tensor, nb: int, hkv: int, cu_seqlens=None,
              max_seqlen: Optional[int] = None) -> dict:
    """Transposes per-query selections into per-block query lists.

    Returns numpy-free plain tensors keyed like the reference's `CSCIndex`:
    col_nnz/col_offsets/order [n_seq,Hkv,nb(+1)], row_indices/head_indices/
    slot_of_pair [n_seq,Hkv,cap]. Within a column entries are ordered by
    (query head, row) ascending. Rows are batch-local (padded) or packed token
    indices (packed); `order` is a stable descending sort of col_nnz.
    """
    bq, hq, t, slots = block_idx.shape
    g = hq // hkv
    if cu_seqlens is None:
        seqs = [(b, 0, t) for b in range(bq)]
        rows_cap = t
    else:
        seqs = [(0, lo, hi) for lo, hi in _spans(t, cu_seqlens)]
        rows_cap = max_seqlen if max_seqlen is not None else max(hi - lo for _, lo, hi in seqs)
    n_seq = len(seqs)
    cap = g * rows_cap * slots
    col_nnz = torch.zeros(n_seq, hkv, nb, dtype=torch.int32)
    col_off = torch.zeros(n_seq, hkv, nb + 1, dtype=torch.int32)
    rows_o = torch.zeros(n_seq, hkv, cap, dtype=torch.int32)
    heads_o = torch.zeros(n_seq, hkv, cap, dtype=torch.int32)
    slots_o = torch.zeros(n_seq, hkv, cap, dtype=torch.int32)
    for si, (b, lo, hi) in enumerate(seqs):
        for hk in range(hkv):
            sub = block_idx[b, hk * g:(hk + 1) * g, lo:hi]              # [g, s, slots]
            gi, ri, ki = torch.nonzero(sub >= 0, as_tuple=True)
            blk = sub[gi, ri, ki].to(torch.int64)
            key = (blk * g + gi) * (hi - lo) + ri
            perm = torch.argsort(key, stable=True)
            n = perm.numel()
            rows_o[si, hk, :n] = (ri[perm] + lo).to(torch.int32)
            heads_o[si, hk, :n] = (gi[perm] + hk * g).to(torch.int32)
            slots_o[si, hk, :n] = ki[perm].to(torch.int32)
            cnt = torch.bincount(blk, minlength=nb)[:nb]
            col_nnz[si, hk] = cnt.to(torch.int32)
            col_off[si, hk, 1:] = cnt.cumsum(0).to(torch.int32)
    order = torch.argsort(col_nnz.to(torch.int64), dim=-1, descending=True,
                          stable=True).to(torch.int32)
    return dict(col_nnz=col_nnz, col_offsets=col_off, row_indices=rows_o,
                head_indices=heads_o, slot_of_pair=slots_o, order=order)


# --------------------------------------------------------------------------
# closed forms used by the benchmark's accounting (reference: bench/suite.py:66-126)
# --------------------------------------------------------------------------

def attended_pairs(seq_len: int, block_size: int, top_k: int) -> int:
    """Number of attended (query, key) pairs per query head for one sequence,
    own block causally trimmed, with the default flags."""
    total = 0
    for pos0 in range(0, seq_len, block_size):
        j = pos0 // block_size
        rows = min(block_size, seq_len - pos0)
        total += rows * (rows + 1) // 2                    # own block, causal
        total += rows * min(j, top_k - 1) * block_size     # past blocks are full
    return total


def selected_pairs(seq_len: int, block_size: int, top_k: int) -> int:
    """(query, block) pairs per query head for one sequence, default flags."""
    total = 0
    for pos0 in range(0, seq_len, block_size):
        j = pos0 // block_size
        rows = min(block_size, seq_len - pos0)
        total += rows * (1 + min(j, top_k - 1))
    return total
