"""The launch table, host side (reference: src/moba/kernels/tuning.py:335-409, which
looks launch parameters up in a baked table keyed by shape; its autotuner has no
counterpart here).

`launch_plan` asks the library what it would run for a problem: which kernel
family each stage takes, the tile plan of the tensor-core kernels (one per
head_dim), how the transpose cuts the rows and how the scheduler cuts the columns.
It is a constant-time lookup on the problem record: nothing is measured and no
device is touched, so it can be called on a machine without a GPU.
"""

from typing import Optional

import torch

from moba_triton_b200 import _lib
from moba_triton_b200.config import MoBAConfig

_PATH_NAMES = {_lib.PATH_PORTABLE: "portable", _lib.PATH_TCGEN05: "tcgen05"}


def launch_plan(q_shape, kv_heads: int, dtype: torch.dtype, cfg: MoBAConfig, cu_seqlens=None,
                max_seqlen: Optional[int] = None) -> dict:
    """{field: value} of `moba_b200_plan` for q of `q_shape` = (B, S, Hq, D); the three
    `*_path` entries are given by name. Raises ValueError for a problem the library rejects."""
    prob = _lib.make_problem(tuple(q_shape), kv_heads, dtype, cfg, cu_seqlens, max_seqlen)
    plan = _lib.Plan()
    _lib.check(_lib.load().moba_b200_launch_plan(prob, plan), "launch_plan")
    out = {name: int(getattr(plan, name)) for name, _ in plan._fields_}
    for stage in ("gate_path", "fwd_path", "bwd_path"):
        out[stage] = _PATH_NAMES[out[stage]]
    return out
