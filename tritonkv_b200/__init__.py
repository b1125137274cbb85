"""tritonkv_b200: single-token decode attention on a packed 2/4-bit KV cache for
NVIDIA B200 (sm_100a).

The public surface mirrors the one hot path of the reference project:

* :mod:`tritonkv_b200.quantize` -- ``QuantizedTensor``, ``quantize_kv``, ``pack_codes`` ...
* :mod:`tritonkv_b200.kernels`  -- ``fused_decode_attention``, ``fp16_decode_attention``,
  ``triton_available``, ``pick_num_splits``

All compute runs in hand-written CUDA kernels behind a C ABI
(``include/tritonkv_b200.h`` -> ``libtritonkv_b200.so``); there is no CPU path.
"""

from . import quantize  # noqa: F401
from . import kernels  # noqa: F401
from .kernels import (  # noqa: F401
    fused_decode_attention,
    fp16_decode_attention,
    triton_available,
    pick_num_splits,
    combine_splits,
)
from .quantize import (  # noqa: F401
    SUPPORTED_BITS,
    QuantizedTensor,
    pack_codes,
    unpack_codes,
    quantize_groupwise,
    dequantize_groupwise,
    quantize_kv,
    roundtrip_error,
)

from .serving import GraphedDecodeStep  # noqa: F401,E402

__version__ = "0.1.0"
