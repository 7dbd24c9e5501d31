"""moda_b200 — B200 (sm_100a) implementation of the MoDA attention operators.

Drop-in for ``fla.ops.moda`` of hustvl/MoDA (libs/moda_triton/fla/ops/moda/__init__.py:5-29)
plus ``fla.ops.moda.fda_v12.parallel_fda``; see ``moda_b200.ops``.
"""
from .ops import (  # noqa: F401
    CHUNK_VISIBLE_QUERY_ROWS,
    fold_qkv,
    last_launch_count,
    moda_attention,
    parallel_fda,
    parallel_fda_bwd,
    parallel_fda_fwd,
    parallel_moda,
    parallel_moda_bwd,
    parallel_moda_chunk_visible,
    parallel_moda_chunk_visible_bwd,
    parallel_moda_chunk_visible_fwd,
    parallel_moda_fwd,
    set_kernel_path,
    tensor_pipe_rates,
)
from .depth_cache import DepthKVCache  # noqa: F401
from ._cabi import (  # noqa: F401
    MODE_CAUSAL, MODE_CHUNK_VISIBLE, MODE_DEPTH_ONLY, MODE_NONCAUSAL,
    PATH_AUTO, PATH_SIMT_MMA, PATH_TCGEN05, PATH_TCGEN05_ONE_TILE, PATH_TCGEN05_TWO_TILES, PATH_TCGEN05_FUSED_BWD,
    ModaLibraryError,
    device_status,
)

__all__ = [
    "parallel_moda", "parallel_moda_fwd", "parallel_moda_bwd",
    "parallel_moda_chunk_visible", "parallel_moda_chunk_visible_fwd", "parallel_moda_chunk_visible_bwd",
    "parallel_fda", "parallel_fda_fwd", "parallel_fda_bwd",
    "moda_attention", "fold_qkv", "DepthKVCache", "set_kernel_path", "last_launch_count", "device_status", "tensor_pipe_rates",
]
