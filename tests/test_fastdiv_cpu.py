"""The multiply-and-shift division of the tensor-core kernels' index arithmetic (csrc/conv_tc.cu: FastDiv): the
constants as the host forms them, checked against integer division over the whole range the kernels use it on
(numerators below 2^31), at the numerators where a rounding error would show first."""
import random


def fastdiv_make(d):
    s = 0
    while (1 << s) < d:
        s += 1
    return ((1 << (31 + s)) // d) + 1, 31 + s


def test_constants_fit_and_divide_exactly():
    rnd = random.Random(5)
    divisors = list(range(1, 300)) + [2 ** k + e for k in range(8, 31) for e in (-1, 0, 1)] + [2 ** 31 - 1] + [rnd.randrange(1, 2 ** 31) for _ in range(300)]
    top = 2 ** 31 - 1
    for d in divisors:
        if not 1 <= d <= top:
            continue
        mul, shift = fastdiv_make(d)
        assert mul < 2 ** 32 and shift <= 62, (d, mul, shift)
        numerators = {0, 1, d - 1, d, d + 1, top, top - 1, top // d * d, max(0, top // d * d - 1)}
        numerators |= {min(top, k * d + e) for k in (2, 3, 1000, top // d // 2) for e in (-1, 0, 1) if k * d + e >= 0}
        numerators |= {rnd.randrange(0, top + 1) for _ in range(20)}
        for n in numerators:
            assert (n * mul) >> shift == n // d, (n, d)
