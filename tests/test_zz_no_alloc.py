"""The transpose entry point for callers that cannot allocate device memory
(`moba_b200_transpose_noalloc`): its scratch is an array built into the library
instead of a caller buffer. Called here straight through the C ABI and compared,
entry by entry, with `moba_b200_transpose` on the same selections -- twice in a
row, because every call reuses the same array and must not depend on what the
previous call left in it. The file name keeps this test last in collection
order; it also passes when run alone in a fresh process."""

import ctypes

import pytest
import torch

import moba_triton_b200 as moba
from moba_triton_b200 import _lib

from conftest import make_qkv

pytestmark = pytest.mark.gpu


def _transpose(noalloc, prob, block_idx, cu, hkv, nb, cap, n_seq, dev):
    i32 = dict(device=dev, dtype=torch.int32)
    # poisoned outputs: everything that matters must be written by the call
    lib = _lib.load()
    per_row = lib.moba_b200_work_items_per_row(prob)
    outs = [torch.full((n_seq, hkv, nb), -7, **i32), torch.full((n_seq, hkv, nb + 1), -7, **i32),
            torch.full((n_seq, hkv, nb), -7, **i32), torch.full((n_seq, hkv, cap), -7, **i32),
            torch.full((n_seq, hkv, cap), -7, **i32), torch.full((n_seq, hkv, cap), -7, **i32),
            torch.full((n_seq, hkv, per_row, 4), -7, **i32)]
    args = [prob, _lib.ptr(block_idx), _lib.ptr(cu)] + [_lib.ptr(t) for t in outs]
    if noalloc:
        rc = lib.moba_b200_transpose_noalloc(*args, _lib.stream_ptr(dev))
    else:
        nbytes = lib.moba_b200_transpose_scratch_bytes(prob)
        scratch = torch.empty((max(nbytes, 4),), device=dev, dtype=torch.uint8)
        rc = lib.moba_b200_transpose(*args, _lib.ptr(scratch), scratch.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "transpose")
    torch.cuda.synchronize()
    return outs


@pytest.mark.parametrize("shape,hkv,bs,top_k,cu", [
    ((1, 4096, 4, 64), 2, 128, 8, None),
    ((1, 1024, 4, 64), 2, 64, 3, [0, 300, 428, 1000, 1024]),
])
def test_noalloc_transpose_matches_the_caller_scratch_entry_point(shape, hkv, bs, top_k, cu, device):
    cfg = moba.MoBAConfig(bs, top_k)
    q, k, _ = make_qkv(shape, hkv, dtype=torch.bfloat16, seed=23)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=device)
    longest = None if cu is None else max(b - a for a, b in zip(cu[:-1], cu[1:]))
    qd, kd = q.to(device), k.to(device)
    kbar = moba.pool_blocks(kd, cfg, cu_seqlens=cu_t, max_seqlen=longest)
    block_idx = moba.gate_select(qd, kbar, cfg, cu_seqlens=cu_t, max_seqlen=longest)
    prob = _lib.make_problem(shape, hkv, torch.bfloat16, cfg, cu_t, longest)
    n_seq, nb = kbar.shape[0], kbar.shape[2]
    cap = (shape[2] // hkv) * (longest or shape[1]) * cfg.slots_per_query
    want = _transpose(False, prob, block_idx, cu_t, hkv, nb, cap, n_seq, device)
    totals = want[0].sum(dim=-1)
    # another selection of the same shape: run between the compared calls, it leaves foreign
    # counts in the built-in array, which the next call must not see
    q2, k2, _ = make_qkv(shape, hkv, dtype=torch.bfloat16, seed=24)
    other_idx = moba.gate_select(q2.to(device), moba.pool_blocks(k2.to(device), cfg, cu_seqlens=cu_t, max_seqlen=longest),
                                 cfg, cu_seqlens=cu_t, max_seqlen=longest)
    assert not torch.equal(other_idx, block_idx)
    for attempt in range(2):                      # two calls in a row share the built-in array
        if attempt == 1:
            _transpose(True, prob, other_idx, cu_t, hkv, nb, cap, n_seq, device)
        got = _transpose(True, prob, block_idx, cu_t, hkv, nb, cap, n_seq, device)
        for name, g, w in zip(("col_nnz", "col_offsets", "order"), got[:3], want[:3]):
            assert torch.equal(g, w), f"{name} differs on call {attempt + 1}"
        for si in range(n_seq):
            for h in range(hkv):
                n = int(totals[si, h])
                for name, g, w in zip(("row_indices", "head_indices", "slot_of_pair"), got[3:6], want[3:6]):
                    assert torch.equal(g[si, h, :n], w[si, h, :n]), f"{name} differs on call {attempt + 1}"
        # work items: same cuts; partial-slot numbers only name scratch memory and may differ
        assert torch.equal(got[6][..., :3], want[6][..., :3]), f"work items differ on call {attempt + 1}"
        assert torch.equal(got[6][..., 3].clamp(max=0), want[6][..., 3].clamp(max=0))


def test_noalloc_transpose_refuses_problems_beyond_its_built_in_scratch(device):
    cfg = moba.MoBAConfig(128, 8)
    shape, hkv = (1, 262144, 8, 64), 8            # needs 16 MiB of scratch, the array holds 8 MiB
    prob = _lib.make_problem(shape, hkv, torch.bfloat16, cfg)
    lib = _lib.load()
    assert lib.moba_b200_transpose_scratch_bytes(prob) > 8 << 20
    dummy = torch.zeros(16, device=device, dtype=torch.int32)
    p = _lib.ptr(dummy)
    rc = lib.moba_b200_transpose_noalloc(prob, p, None, p, p, p, p, p, p, p, _lib.stream_ptr(device))
    assert rc == -2
    assert b"built-in" in lib.moba_b200_last_error()


def test_noalloc_transpose_leaves_device_memory_untouched(device):
    """The call itself must neither allocate nor free device memory: the free-memory figure
    of the driver is the same before and after (outputs are allocated beforehand, and the
    first call, which looks up the built-in array's address, has already happened)."""
    cfg = moba.MoBAConfig(128, 8)
    shape, hkv = (1, 4096, 4, 64), 2
    q, k, _ = make_qkv(shape, hkv, dtype=torch.bfloat16, seed=23)
    kbar = moba.pool_blocks(k.to(device), cfg)
    block_idx = moba.gate_select(q.to(device), kbar, cfg)
    prob = _lib.make_problem(shape, hkv, torch.bfloat16, cfg)
    nb, cap = kbar.shape[2], (shape[2] // hkv) * shape[1] * cfg.slots_per_query
    i32 = dict(device=device, dtype=torch.int32)
    lib = _lib.load()
    outs = [torch.empty((1, hkv, nb), **i32), torch.empty((1, hkv, nb + 1), **i32), torch.empty((1, hkv, nb), **i32),
            torch.empty((1, hkv, cap), **i32), torch.empty((1, hkv, cap), **i32), torch.empty((1, hkv, cap), **i32),
            torch.empty((1, hkv, lib.moba_b200_work_items_per_row(prob), 4), **i32)]
    args = [prob, _lib.ptr(block_idx), None] + [_lib.ptr(t) for t in outs] + [_lib.stream_ptr(device)]
    _lib.check(lib.moba_b200_transpose_noalloc(*args), "transpose")      # first call on this device
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(device)
    reserved_before = torch.cuda.memory_reserved(device)
    for _ in range(3):
        _lib.check(lib.moba_b200_transpose_noalloc(*args), "transpose")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(device)
    assert torch.cuda.memory_reserved(device) == reserved_before
    assert free_after == free_before, "the call changed the amount of free device memory"
