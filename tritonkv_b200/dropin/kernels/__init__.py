"""Drop-in package named like the reference's ``kernels`` (kernels/__init__.py:1-6)."""

from .fused_decode_attn import (  # noqa: F401
    fused_decode_attention,
    triton_available,
    pick_num_splits,
)
from .fp16_decode_attn import fp16_decode_attention  # noqa: F401
