"""The reference's own correctness suite (test_correctness.py, unmodified) run against this
package through the drop-in module names: ``quantize`` and ``kernels.fused_decode_attn``
resolve to ``tritonkv_b200/dropin``, ``reference`` (its fp32 oracle and input generator) to
the reference's own file.  Runs where ``baseline/fetch_ref.py`` has placed the reference's
files under the git-ignored ``baseline/_ref``; skipped elsewhere.

Five of its tests quantise CPU tensors (test_correctness.py:78-134: pack/unpack round trip,
half-step bound, constant group, 4-bit beats 2-bit, effective bits).  This package has no CPU
path by design, so they are deselected here; the same properties are asserted on CUDA
tensors in tests/test_gpu_quantize.py."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
CPU_ONLY = ("pack_unpack_roundtrip or quant_error_within_half_step or constant_group_is_exact or "
            "higher_bits_are_more_accurate or effective_bits_accounts_for_metadata")


def test_reference_suite_passes_through_the_dropin_modules():
    suite = os.path.join(REF, "test_correctness.py")
    if not os.path.isfile(suite):
        pytest.skip("baseline/_ref/test_correctness.py is absent (baseline/fetch_ref.py was not run)")
    env = dict(os.environ)
    # drop-in names first, then this repository, then the reference (for `reference`).  The
    # child runs FROM the drop-in directory: `python -m` puts the working directory at the
    # head of sys.path, and from baseline/_ref that would be the reference's own modules.
    dropin = os.path.join(ROOT, "tritonkv_b200", "dropin")
    env["PYTHONPATH"] = os.pathsep.join([dropin, ROOT, REF])
    r = subprocess.run([sys.executable, "-m", "pytest", suite, "-q", "-x", "-p", "no:cacheprovider",
                        "--import-mode=importlib", "--rootdir", REF, "-k", f"not ({CPU_ONLY})"],
                       capture_output=True, text=True, env=env, cwd=dropin, timeout=1500)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "failed" not in r.stdout, tail
    # the kernels under test were this package's: the drop-in reports the CUDA library
    probe = subprocess.run([sys.executable, "-c",
                            "from kernels.fused_decode_attn import triton_available as t; print(t()[1])"],
                           capture_output=True, text=True, env=env, cwd=dropin, timeout=300)
    assert "tritonkv_b200" in probe.stdout, probe.stdout + probe.stderr
