"""Backend adapter with the interface of the reference's `OursBackend`
(reference: implementations/ours.py:32-159, protocol implementations/base.py:21-83).

An instance can be handed to the reference's `register()`; its harness then
drives this engine through the same four calls it uses for every backend.
"""

import torch

import moba_triton_b200 as moba
from moba_triton_b200.device import device_is_supported

SUPPORTED_DTYPES = (torch.bfloat16, torch.float16, torch.float32)


class B200Backend:
    """`name`, `vendored`, `computes_moba`, `is_available`, `forward`,
    `forward_grad`, `selection` -- the attributes and methods of the protocol."""

    name = "ours_b200"
    vendored = False
    computes_moba = True

    def is_available(self, cfg) -> tuple:
        """(available, reason); never raises."""
        try:
            ok, why = device_is_supported()
            if not ok:
                return False, why
            if cfg.dtype not in SUPPORTED_DTYPES:
                return False, f"unsupported dtype {cfg.dtype}"
            if cfg.block_size < 16:
                return False, f"block_size {cfg.block_size} below the minimum of 16"
            from moba_triton_b200 import _lib
            _lib.load()
            return True, ""
        except Exception as exc:          # the protocol asks for a reason, not an exception
            return False, f"{type(exc).__name__}: {exc}"

    def forward(self, q, k, v, cfg):
        return moba.moba_forward(q, k, v, cfg)

    def forward_grad(self, q, k, v, cfg):
        return moba.moba_attention(q, k, v, cfg)

    def selection(self, q, k, cfg):
        return moba.csc_to_mask(moba.build_csc_fused(q, k, cfg), q.shape[1])
