"""The helion_mlir_utils operator set, B200-native.

The 30 names of the reference's ``helion_mlir_utils/__init__.py`` with the same
signatures, plus ``layer_norm``, ``rms_norm``, ``matmul_blocked`` and the fused
epilogue helpers. Every operator enqueues hand-written sm_100a kernels from
``libb200ops.so`` on the caller's current CUDA stream.
"""

from __future__ import annotations

from .attention import attention
from .elementwise import leaky_relu
from .elementwise import relu
from .elementwise import scalar_mul
from .host_io import stream_rows
from .epilogues import gelu_tanh
from .epilogues import leaky_relu_epilogue
from .kernels import per_config
from .linear import CACHE_PREPACKED_WEIGHTS_ENV
from .linear import AffineLinearCache
from .linear import LinearCache
from .linear import cache_prepacked_weights
from .linear import linear
from .linear import linear_affine
from .matmul import bmm
from .matmul import identity_epilogue
from .matmul import matmul
from .matmul import matmul_blocked
from .matmul import matmul_host
from .matmul import matmul_prepacked_b
from .matmul import matmul_prepacked_b_affine
from .matmul import pack_a_blocked
from .matmul import pack_a_blocked_t
from .matmul import pack_b_blocked
from .matmul import pack_b_blocked_t
from .matmul import pack_b_blocked_vnni
from .matmul import pack_b_blocked_vnni_t
from .matmul import pack_b_vnni_t
from .matmul import pad_2d
from .matmul import prepacked_b_call
from .matmul import supports
from .matmul import tall_output_tiles
from .matmul import unpack_b_to_nk
from .matmul import vnni_panel
from .matmul import whole_row_tiles
from .normalization import add_extra
from .normalization import group_norm
from .normalization import layer_norm
from .normalization import mul_extra
from .normalization import rms_norm
from .normalization import softmax
from .reduction import column_sum
from .reduction import matvec
from .reduction import row_dot
from .reduction import row_sum
from .reduction import supports_matvec
from .sharding import column_sharded_linear
from .sharding import gather_rows
from .sharding import row_sharded
from .sharding import shard_bounds
from .sharding import shard_rows
from .tuning import tune_matmul

__all__ = [
    "CACHE_PREPACKED_WEIGHTS_ENV",
    "AffineLinearCache",
    "LinearCache",
    "add_extra",
    "attention",
    "bmm",
    "cache_prepacked_weights",
    "column_sharded_linear",
    "column_sum",
    "gather_rows",
    "gelu_tanh",
    "group_norm",
    "identity_epilogue",
    "layer_norm",
    "leaky_relu",
    "leaky_relu_epilogue",
    "linear",
    "linear_affine",
    "matmul",
    "matmul_blocked",
    "matmul_host",
    "matmul_prepacked_b",
    "matmul_prepacked_b_affine",
    "matvec",
    "mul_extra",
    "pack_a_blocked",
    "pack_a_blocked_t",
    "pack_b_blocked",
    "pack_b_blocked_t",
    "pack_b_blocked_vnni",
    "pack_b_blocked_vnni_t",
    "pack_b_vnni_t",
    "pad_2d",
    "per_config",
    "prepacked_b_call",
    "relu",
    "rms_norm",
    "row_dot",
    "row_sharded",
    "row_sum",
    "scalar_mul",
    "shard_bounds",
    "shard_rows",
    "softmax",
    "stream_rows",
    "tune_matmul",
    "supports",
    "supports_matvec",
    "tall_output_tiles",
    "unpack_b_to_nk",
    "vnni_panel",
    "whole_row_tiles",
]

# HELION_MLIR_TRACE_CALLS=1: every operator reports the first call with each kind of
# operands and an at-exit summary counts the calls. Unset: nothing is wrapped.
_OPERATORS = [
    "attention", "bmm", "column_sum", "group_norm", "layer_norm", "leaky_relu", "linear", "linear_affine", "matmul",
    "matmul_blocked", "matmul_host", "matmul_prepacked_b", "matmul_prepacked_b_affine", "matvec", "pack_a_blocked",
    "pack_a_blocked_t", "pack_b_blocked", "pack_b_blocked_t", "pack_b_blocked_vnni", "pack_b_blocked_vnni_t",
    "pack_b_vnni_t", "pad_2d", "relu", "rms_norm", "row_dot", "row_sum", "scalar_mul", "softmax", "stream_rows",
]


def _install_tracing() -> None:
    from helion_mlir_backend import call_trace

    call_trace.install(globals(), _OPERATORS)


_install_tracing()
