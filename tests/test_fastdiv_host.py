"""The multiply-high division the scheduler uses for divisors fixed per launch
(``make_fastdiv`` / ``fast_div`` in ``tritonkv_b200/csrc/tkv_splitk_driver.cuh``), restated in
Python integers: ``l = ceil(log2 d)``, ``m = floor(2^32 (2^l - d) / d) + 1`` and
``n // d == (mulhi32(n, m) + n) >> l`` for every ``0 <= n < 2^31``, with the 32-bit sum never
overflowing.  (The kernels only ever divide tile, unit and CTA indices, all below 2^31.)"""

import random

import pytest


def make_fastdiv(d: int):
    d = max(d, 1)
    l = 0
    while (1 << l) < d:
        l += 1
    m = ((1 << 32) * ((1 << l) - d)) // d + 1
    return m, l


def fast_div(n: int, m: int, l: int) -> int:
    hi = (n * m) >> 32          # __umulhi
    s = hi + n
    assert s < (1 << 32)        # the kernel's 32-bit addition does not wrap
    return s >> l


@pytest.mark.parametrize("seed", [0, 1])
def test_fast_division_is_exact_below_two_to_the_31(seed):
    rng = random.Random(seed)
    divisors = list(range(1, 2049)) + [rng.randrange(1, 1 << 31) for _ in range(2000)] + [(1 << 31) - 1]
    for d in divisors:
        m, l = make_fastdiv(d)
        assert m < (1 << 32)
        edge = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, 3 * d - 1, (1 << 31) - 1, (1 << 31) - 2]
        for n in edge + [rng.randrange(0, 1 << 31) for _ in range(64)]:
            if 0 <= n < (1 << 31):
                assert fast_div(n, m, l) == n // d, (n, d)


def test_divisor_one_and_zero_are_the_identity():
    for d in (0, 1):
        m, l = make_fastdiv(d)
        assert (m, l) == (1, 0)
        assert fast_div(123456789, m, l) == 123456789
