"""``kernels.fused_decode_attn`` of the reference, served by the CUDA implementation."""

from tritonkv_b200.kernels.fused_decode_attn import (  # noqa: F401
    LOG2E,
    combine_splits,
    fused_decode_attention,
    pick_num_splits,
    triton_available,
)
