"""Generates tests/golden/*.npz by running the reference's own oracle.

Run where the reference checkout is importable (it is not available on the GPU
machines, which is why the vectors are committed):

    MOBA_REFERENCE_SRC=/path/to/reference/src python tests/golden/make_golden.py

Every case stores its inputs bit-exactly (as bfloat16 bit patterns -- all
inputs are bfloat16-representable so the same numbers can be replayed in
float64, float32 and bfloat16), the reference `moba.naive.moba_selection` mask,
the reference `moba_attention_naive` output evaluated in float64 with that
mask, and the float64 autograd gradients for a stored upstream gradient.
"""

import os
import sys

import numpy as np
import torch

REF = os.environ.get("MOBA_REFERENCE_SRC")
if not REF:
    raise SystemExit("set MOBA_REFERENCE_SRC to the `src` directory of a ZuricZ/moba-triton checkout")
sys.path.insert(0, REF)

from moba.config import MoBAConfig                       # noqa: E402  (reference)
from moba.naive import moba_attention_naive, moba_selection   # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name, q shape [B,S,Hq,D], Hkv, block, top_k, sel dtype, cu_seqlens, flags, seed
CASES = [
    ("mha_f32_s256_bs32_k4", (1, 256, 2, 64), 2, 32, 4, torch.float32, None, {}, 0),
    ("mha_bf16_s512_bs64_k4", (1, 512, 2, 64), 2, 64, 4, torch.bfloat16, None, {}, 1),
    ("batch2_f32_s128_bs16_k3", (2, 128, 2, 64), 2, 16, 3, torch.float32, None, {}, 2),
    ("gqa_f32_s192_bs32_k3", (1, 192, 4, 64), 2, 32, 3, torch.float32, None, {}, 3),
    ("tail_f32_s200_bs32_k4", (1, 200, 2, 64), 2, 32, 4, torch.float32, None, {}, 4),
    ("varlen_f32_bs16_k3", (1, 212, 2, 64), 2, 16, 3, torch.float32, [0, 80, 128, 192, 212], {}, 5),
    ("varlen_gqa_bf16_bs16_k3", (1, 212, 4, 64), 2, 16, 3, torch.bfloat16, [0, 80, 128, 192, 212], {}, 6),
    ("nocurrent_f32_s256_bs32_k2", (1, 256, 2, 64), 2, 32, 2, torch.float32, None,
     {"always_select_current": False}, 7),
    ("extra_slot_f32_s256_bs32_k2", (1, 256, 2, 64), 2, 32, 2, torch.float32, None,
     {"top_k_includes_current": False}, 8),
    ("ties_f32_s256_bs32_k4", (1, 256, 2, 64), 2, 32, 4, torch.float32, None, {"ties": True}, 9),
    ("d128_bf16_s256_bs128_k2", (1, 256, 1, 128), 1, 128, 2, torch.bfloat16, None, {}, 10),
]


# cases that pin selection and the forward only (no gradients stored). The
# no-own-block case is here because the reference oracle's autograd returns NaN
# for every gradient once any query has an empty selection.
SELECTION_ONLY = {"batch2_f32_s128_bs16_k3", "extra_slot_f32_s256_bs32_k2",
                  "ties_f32_s256_bs32_k4", "nocurrent_f32_s256_bs32_k2"}


def bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    for name, shape, hkv, bs, top_k, sel_dtype, cu, flags, seed in CASES:
        flags = dict(flags)
        ties = flags.pop("ties", False)
        g = torch.Generator().manual_seed(seed)
        b, s, hq, d = shape
        q = torch.randn(shape, generator=g).to(torch.bfloat16)
        k = torch.randn((b, s, hkv, d), generator=g).to(torch.bfloat16)
        v = torch.randn((b, s, hkv, d), generator=g).to(torch.bfloat16)
        do = (torch.randn(shape, generator=g) * 0.1).to(torch.bfloat16)
        if ties:
            # every block of head 0 has the same keys, so all its gate scores tie
            k[:, :, 0] = k[:, :bs, 0].repeat(1, s // bs, 1)
        cfg = MoBAConfig(block_size=bs, top_k=top_k, dtype=sel_dtype, **flags)
        cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)

        mask = moba_selection(q.to(sel_dtype), k.to(sel_dtype), cfg, cu_seqlens=cu_t)

        q64, k64, v64 = (t.to(torch.float64).requires_grad_(True) for t in (q, k, v))
        out = moba_attention_naive(q64, k64, v64, cfg, selected=mask, cu_seqlens=cu_t)
        live = ~torch.isnan(out.detach())          # rows with no selected block are NaN
        (torch.where(live, out, torch.zeros_like(out)) * do.to(torch.float64)).sum().backward()

        low = moba_attention_naive(q.to(sel_dtype), k.to(sel_dtype), v.to(sel_dtype), cfg,
                                   selected=mask, cu_seqlens=cu_t)

        extra = {}
        if sel_dtype == torch.bfloat16:
            extra["out_low"] = bits(low)
        if name not in SELECTION_ONLY:
            extra.update(do=bits(do),
                         dq=q64.grad.to(torch.float32).numpy(),
                         dk=k64.grad.to(torch.float32).numpy(),
                         dv=v64.grad.to(torch.float32).numpy())
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            q=bits(q), k=bits(k), v=bits(v),
            mask=np.packbits(mask.numpy()), mask_shape=np.array(mask.shape),
            out=out.detach().to(torch.float32).numpy(),
            **extra,
            meta=np.array([bs, top_k, hkv,
                           int(cfg.always_select_current), int(cfg.top_k_includes_current),
                           {torch.float32: 0, torch.bfloat16: 1}[sel_dtype]]),
            cu=np.array(cu if cu is not None else [], dtype=np.int32),
        )
        print(f"{name}: pairs={int(mask.sum())} out|max|={float(torch.nan_to_num(out.detach()).abs().max()):.3f}")


if __name__ == "__main__":
    main()
