"""Drop-in module named like the reference's ``quantize.py``: put this directory ahead of
the reference checkout on ``sys.path`` and ``from quantize import ...`` resolves to the
CUDA implementation."""

from tritonkv_b200.quantize import *  # noqa: F401,F403
from tritonkv_b200.quantize import (  # noqa: F401
    SUPPORTED_BITS,
    QuantizedTensor,
    _check_bits,
    _META_BITS_PER_GROUP,
    pack_codes,
    unpack_codes,
    quantize_groupwise,
    dequantize_groupwise,
    quantize_kv,
    roundtrip_error,
)
