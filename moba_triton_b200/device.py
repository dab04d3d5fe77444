"""Capability checks for the sm_100a engine (reference: src/moba/device.py:48-146)."""

import torch

MIN_CAPABILITY = (10, 0)          # the kernels are built for sm_100a only
MIN_BLOCK_SIZE = 16               # reference: TENSOR_CORE_TILE, src/moba/device.py
CACHE_LINE_BYTES = 128


def check_gathered_head_dim(head_dim: int, itemsize: int):
    """(ok, reason): a gathered query row must be a power-of-two number of
    elements and fill at least one 128-byte line (reference: device.py:96-120)."""
    if head_dim <= 0 or head_dim & (head_dim - 1):
        return False, f"head_dim {head_dim} must be a power of two"
    if head_dim * itemsize < CACHE_LINE_BYTES:
        return False, (f"head_dim {head_dim} gives a {head_dim * itemsize}-byte row, below the "
                       f"{CACHE_LINE_BYTES}-byte cache line")
    return True, ""


def supports_dtype(dtype: torch.dtype):
    """(ok, reason) for a compute dtype on this engine."""
    if dtype in (torch.bfloat16, torch.float16, torch.float32):
        return True, ""
    return False, f"unsupported dtype {dtype}"


def device_is_supported(device=None):
    """(ok, reason): needs a CUDA device of compute capability 10.x."""
    if not torch.cuda.is_available():
        return False, "no CUDA device"
    cap = torch.cuda.get_device_capability(device)
    if cap[0] != MIN_CAPABILITY[0]:
        return False, f"built for sm_100a, found sm_{cap[0]}{cap[1]}"
    return True, ""
