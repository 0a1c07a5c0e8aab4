"""B200-native mixed-bit codebook-quantized MoE expert layer (drop-in for DartMoQ-Qwen3.5).

``format``   packed-weight format: packing, codebooks, rotations, quantiser, mode LUTs
``kernels``  function-level operators over libdmoq (the C ABI in include/dmoq.h)
``moe``      WxA16 / WxA8 / WxFP8 / WxFP4 BitPartitionedGroupMoE modules
``linear``   packed dense Linear layers (shared expert)
``host_io``  pipelined layer calls over pinned host batches
``synth``    seeded synthetic layers of the benchmark shapes
``build``    nvcc build of libdmoq.so
"""
from . import format  # noqa: F401
from .moe import (  # noqa: F401
    MODULE_BY_MODE,
    WxA16BitPartitionedGroupMoE,
    WxA16Weights,
    WxA8BitPartitionedGroupMoE,
    WxFP4BitPartitionedGroupMoE,
    WxFP8BitPartitionedGroupMoE,
)
from .linear import WxA16Linear, WxA8Linear, WxFP8Linear  # noqa: F401

__all__ = [
    "format", "MODULE_BY_MODE", "WxA16Weights", "WxA16BitPartitionedGroupMoE", "WxA8BitPartitionedGroupMoE",
    "WxFP8BitPartitionedGroupMoE", "WxFP4BitPartitionedGroupMoE", "WxA16Linear", "WxA8Linear", "WxFP8Linear",
]
