"""Backward of the MoBA forward (reference: src/moba/kernels/moba_bwd.py:454-579)."""

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.gqa import head_group_size
from moba_triton_b200.kernels.moba_fwd import _check_index, _problem
from moba_triton_b200.kernels.routing import CSCIndex


def moba_backward(dout, q, k, v, out, lse, part_lse, cfg: MoBAConfig, index: CSCIndex,
                  causal: bool = True, dq=None, delta=None):
    """Returns (dq, dk, dv) shaped like q, k, v. `lse` is the forward's global
    log2-sum-exp [B,H,S]; `part_lse` the forward's per-slot buffer, read only as
    the written-slot marker. dk/dv are already summed over the query heads that
    share a kv head; the routing receives no gradient.

    With an index of a query window (`index.window`), `part_lse` holds the window's rows,
    only those rows of the given `dq` are written, and dk/dv are the window's contribution.
    `delta` (rowsum(out * dout) [B,H,S]) is computed unless passed in."""
    _lib.require_cuda(dout, q, k, v, out, lse, part_lse)
    head_group_size(q.shape[2], k.shape[2])
    _check_index(q, k, cfg, index)
    q, k, v, dout, out = (t.contiguous() for t in (q, k, v, dout, out))
    if dout.dtype != q.dtype:
        dout = dout.to(q.dtype)
    b, s, hq, d = q.shape
    prob = _problem(q, k, cfg, index, causal)
    if dq is None:
        dq = torch.empty_like(q)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    if delta is None:
        delta = torch.empty((b, hq, s), device=q.device, dtype=torch.float32)
    rows = s if index.window is None else index.window[1]
    dq_part = torch.empty((b, hq, rows, index.max_slots, d), device=q.device, dtype=q.dtype)
    # float32 dK/dV partials of the columns the scheduler cut into several work items
    dkv_scratch = torch.empty((max(16, _lib.load().moba_b200_dkv_scratch_bytes(prob)),), device=q.device, dtype=torch.uint8)
    _lib.call("moba_b200_bwd", q.device, "moba_backward",
              prob, _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse),
              _lib.ptr(part_lse), index.c_struct(), _lib.ptr(index.cu_seqlens), _lib.ptr(delta),
              _lib.ptr(dq_part), _lib.ptr(dkv_scratch), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv))
    return dq, dk, dv
