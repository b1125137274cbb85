"""With ``tritonkv_b200/dropin`` first on sys.path, the reference's import statements
(test_correctness.py:30-44, benchmark.py:51-52 of the reference) resolve to this package."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_import_lines_resolve_to_the_cuda_package():
    code = (
        "from quantize import SUPPORTED_BITS, dequantize_groupwise, pack_codes, quantize_groupwise, "
        "quantize_kv, unpack_codes, QuantizedTensor\n"
        "from kernels.fused_decode_attn import fused_decode_attention, triton_available\n"
        "from kernels.fp16_decode_attn import fp16_decode_attention\n"
        "from kernels import fused_decode_attention as f2, pick_num_splits\n"
        "import tritonkv_b200\n"
        "assert fused_decode_attention is tritonkv_b200.fused_decode_attention is f2\n"
        "assert QuantizedTensor is tritonkv_b200.QuantizedTensor\n"
        "assert quantize_kv.__module__ == 'tritonkv_b200.quantize'\n"
        "print('ok')\n"
    )
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "tritonkv_b200", "dropin"), ROOT])
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env,
                       cwd="/tmp")
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr
