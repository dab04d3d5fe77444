"""The packed-batch boundary on the device: `pack`, `unpack` and `from_nested` are row
gathers run by CUDA kernels through the C ABI. They move bytes, so every comparison is
exact. The cases follow tests/test_packing.py and tests/test_varlen.py of the reference:
prefix masks, masks with holes, an empty row, every supported mask dtype, a round trip
through the attention op."""

import pytest
import torch

import moba_triton_b200 as moba
from moba_triton_b200.varlen import from_nested, pack, unpack

from conftest import make_qkv

pytestmark = pytest.mark.gpu


def _expected_pack(x, mask):
    keep = mask.bool()
    rows = [x[b][keep[b]] for b in range(x.shape[0])]
    lens = [int(r.shape[0]) for r in rows]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return torch.cat(rows, dim=0).unsqueeze(0), cu, max(lens)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("mask_dtype", [torch.bool, torch.int32, torch.int64, torch.float32])
def test_pack_matches_row_selection_and_unpack_inverts_it(dtype, mask_dtype, device):
    g = torch.Generator().manual_seed(3)
    b, s, h, d = 5, 700, 3, 64
    x = torch.randn(b, s, h, d, generator=g).to(dtype)
    lens = [700, 1, 0, 333, 512]                                 # a full row, a single token, an empty row
    mask = (torch.arange(s)[None, :] < torch.tensor(lens)[:, None])
    packed, cu, longest = pack(x.to(device), mask.to(mask_dtype).to(device))
    want, want_cu, want_longest = _expected_pack(x, mask)
    assert cu.dtype == torch.int32 and cu.device.type == "cuda"
    assert cu.tolist() == want_cu and longest == want_longest
    assert packed.shape == want.shape and packed.is_contiguous()
    assert torch.equal(packed.cpu(), want)
    back = unpack(packed, cu, b, s)
    assert torch.equal(back.cpu(), x * mask[:, :, None, None].to(dtype))
    # a wider rectangle pads with zeros; a poisoned allocator must not show through
    wide = unpack(packed, cu, b, s + 50)
    assert torch.equal(wide[:, :s].cpu(), back.cpu()) and not wide[:, s:].any()


def test_pack_keeps_order_under_a_mask_with_holes(device):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(4, 1030, 2, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(4, 1030, generator=g) < 0.6
    packed, cu, longest = pack(x.to(device), mask.to(device))
    want, want_cu, want_longest = _expected_pack(x, mask)
    assert cu.tolist() == want_cu and longest == want_longest
    assert torch.equal(packed.cpu(), want)


def test_from_nested_is_the_packed_form(device):
    g = torch.Generator().manual_seed(5)
    lens = [10, 3, 7, 129]
    x = torch.randn(4, 129, 2, 64, generator=g).to(torch.bfloat16).to(device)
    mask = (torch.arange(129)[None, :] < torch.tensor(lens)[:, None]).to(device)
    packed, cu, longest = pack(x, mask)
    nt = torch.nested.nested_tensor([x[i, :n] for i, n in enumerate(lens)], layout=torch.jagged)
    p2, cu2, l2 = from_nested(nt)
    assert torch.equal(p2, packed) and cu2.tolist() == cu.tolist() and l2 == longest == 129
    assert cu2.dtype == torch.int32


def test_padded_batch_through_pack_op_unpack_equals_per_sequence_runs(device):
    """pack -> attention on the packed batch -> unpack gives, for every sequence, the bits
    of that sequence run alone."""
    cfg = moba.MoBAConfig(128, 4)
    lens = [384, 129, 1000]
    q, k, v = make_qkv((3, 1000, 4, 64), 2, dtype=torch.bfloat16, seed=41)
    qd, kd, vd = (t.to(device) for t in (q, k, v))
    mask = (torch.arange(1000)[None, :] < torch.tensor(lens)[:, None]).to(device)
    qp, cu, longest = pack(qd, mask)
    kp, _, _ = pack(kd, mask)
    vp, _, _ = pack(vd, mask)
    out = unpack(moba.moba_forward(qp, kp, vp, cfg, cu_seqlens=cu, max_seqlen=longest), cu, 3, 1000)
    for i, n in enumerate(lens):
        alone = moba.moba_forward(qd[i:i + 1, :n], kd[i:i + 1, :n], vd[i:i + 1, :n], cfg)
        assert torch.equal(out[i:i + 1, :n], alone)
        assert not out[i, n:].any()
