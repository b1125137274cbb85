"""Decode-attention entry points, same names as the reference's ``kernels`` package
(kernels/__init__.py:1-6)."""

from .fused_decode_attn import (  # noqa: F401
    fused_decode_attention,
    triton_available,
    pick_num_splits,
    combine_splits,
)
from .fp16_decode_attn import fp16_decode_attention  # noqa: F401
from .kivi_decode_attn import KiviCache, kivi_decode_attention, quantize_kv_kivi  # noqa: F401
