"""B200-native MoBA (Mixture of Block Attention) engine.

Drop-in for the `moba` package of ZuricZ/moba-triton on its attention path:
`MoBAConfig`, `moba_attention` (differentiable), `moba_forward`,
`build_csc_fused`, `csc_to_mask`, `CSCIndex`, `pool_blocks`, `gate_select`.
Use it as `import moba_triton_b200 as moba`. All compute happens in
hand-written sm_100a CUDA kernels behind the C ABI of `include/moba_b200.h`;
importing needs no GPU, calling does.
"""

from moba_triton_b200.config import MoBAConfig
from moba_triton_b200.kernels.attention import MoBAAttentionFunction, moba_attention
from moba_triton_b200.kernels.gating import gate_select
from moba_triton_b200.kernels.moba_fwd import (attend_partials, combine_partials,
                                               merge_partials, moba_forward)
from moba_triton_b200.kernels.moba_bwd import moba_backward
from moba_triton_b200.kernels.pooling import pool_blocks
from moba_triton_b200.kernels.routing import (CSCIndex, build_csc_from_indices,
                                              build_csc_fused, csc_to_mask)

__all__ = [
    "MoBAConfig", "moba_attention", "moba_forward", "build_csc_fused", "csc_to_mask",
    "CSCIndex", "pool_blocks", "gate_select", "build_csc_from_indices", "attend_partials",
    "combine_partials", "merge_partials", "moba_backward", "MoBAAttentionFunction",
]
__version__ = "0.1.0"
