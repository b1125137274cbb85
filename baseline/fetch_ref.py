"""Place the reference project's hot-path modules under ``baseline/_ref/`` (git-ignored).

    python baseline/fetch_ref.py /path/to/reference

The reference (PS12007/tritonkv) has no packaging, so "installing" it is copying the five
modules of its decode path, unmodified: ``quantize.py``, ``reference.py`` and
``kernels/{__init__,fused_decode_attn,fp16_decode_attn}.py``, plus its correctness suite
``test_correctness.py``.  ``baseline/_ref/`` is never committed and nothing in
``tritonkv_b200/`` imports it; its users are ``baseline/triton_leg.py``, a separate process
that ``bench.py`` starts to time the reference's own Triton kernels on the same GPU next to
the CUDA kernels of this package, and ``tests/test_gpu_reference_suite.py``, which runs the
reference's test file against the drop-in modules.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = ["quantize.py", "reference.py", "kernels/__init__.py", "kernels/fused_decode_attn.py",
         "kernels/fp16_decode_attn.py",
         # the reference's own correctness suite, run unmodified through the drop-in modules
         # of this package by tests/test_gpu_reference_suite.py
         "test_correctness.py"]


def fetch(ref_root: str) -> str:
    for rel in FILES:
        src = os.path.join(ref_root, rel)
        if not os.path.isfile(src):
            raise FileNotFoundError(f"{src}: not a checkout of the reference project")
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(fetch(sys.argv[1]))
