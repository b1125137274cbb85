"""``kernels.fp16_decode_attn`` of the reference, served by the CUDA implementation."""

from tritonkv_b200.kernels.fp16_decode_attn import fp16_decode_attention  # noqa: F401
