"""Bit-exact decode: the device decoders over all 65,536 codewords and the W_hat kernel against the oracle's
reconstructInner (the reference's own GPU tests of the same: src/hip_tests.zig:24-57, 59-123; W_hat bit-exactness is
the first result requirement: the decoded weights are the bits of the reference)."""
import numpy as np
import pytest
import torch

import turboexl3_b200 as t3
from oracle import binding as ob
from turboexl3_b200 import synth

from gpu_util import bits16, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("codebook", [t3.MUL1, t3.MCG])
@pytest.mark.parametrize("window", [16, 15, 12, 8])
def test_every_codeword(codebook, window):
    got = bits16(t3.codebook_table(t3.Decode(codebook, window)))
    assert np.array_equal(got, ob.decode_table(codebook, window))


@pytest.mark.parametrize("n", [16, 32, 48, 64, 80, 96, 112, 128, 18, 36, 40, 44, 56, 104, 126])
@pytest.mark.parametrize("codebook", [t3.MUL1, t3.MCG])
def test_w_hat_bit_exact_every_rate(n, codebook):
    in_dim, out_dim = 256, 384
    trellis, _, _ = synth.linear(1000 + n, in_dim, out_dim, n)
    for window in (16, 12):
        got = bits16(t3.dequantize(dev(trellis), t3.Decode(codebook, window)))
        want = ob.reconstruct_inner(trellis, in_dim, out_dim, n, codebook, window)
        assert np.array_equal(got, want), (n, codebook, window, int((got != want).sum()))


def test_w_hat_config1_4096x4096_k4():
    """Benchmark config 1: in 4096, out 4096, K = 4, codes from seed 0; W_hat must match bit for bit."""
    trellis, _, _ = synth.linear(0, 4096, 4096, 64)
    got = bits16(t3.dequantize(dev(trellis), t3.Decode.mul1))
    want = ob.reconstruct_inner(trellis, 4096, 4096, 64, ob.MUL1)
    assert np.array_equal(got, want)
    assert t3.device_error() == 0


def test_w_hat_i16_trellis_is_the_same_words():
    trellis, _, _ = synth.linear(5, 128, 128, 64)
    a = bits16(t3.dequantize(dev(trellis)))
    b = bits16(t3.dequantize(dev(trellis.view(np.int16))))
    assert np.array_equal(a, b)
