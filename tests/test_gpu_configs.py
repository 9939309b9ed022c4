"""The benchmark configurations 4 and 5 against the oracle: the hybrid layer with a rate drawn per expert from {2, 3, 4} bits (one
sub-bank a rate, turboexl3_b200.mixed), the large layer's geometry (hidden 7168, width 2048, top-8, sigmoid scores, one
shared expert, K = 2 and K = 4) at decode and prefill rows, and the MLA trunk projections at K = 4. Expert counts are cut
down (the oracle decodes every weight of every expert a row touches on the host); geometry, rates, routing and the kernels'
paths are the configs'. Bars are those of test_gpu_moe / test_gpu_linear."""
import numpy as np
import pytest
import torch

import turboexl3_b200 as t3
from oracle import binding as ob
from turboexl3_b200 import mixed, synth

from gpu_util import check, dev, host_f32, x_as
from test_gpu_moe import check_moe, make_bank

pytestmark = pytest.mark.gpu


def _slot_sum(v: np.ndarray, scores: np.ndarray) -> np.ndarray:
    """ref.moeRow's accumulation (src/core/ref.zig:106): y += score * d, a multiply then an add in f32, slots in order."""
    y = np.zeros((v.shape[0], v.shape[2]), np.float32)
    for k in range(v.shape[1]):
        y = (y + (scores[:, k:k + 1].astype(np.float32) * v[:, k]).astype(np.float32)).astype(np.float32)
    return y


def test_config4_rate_per_expert():
    H, I, E, topk = 2048, 512, 24, 10
    rng = np.random.default_rng(4)
    rates = [16 * int(k) for k in rng.choice([2, 3, 4], E)]
    buckets = mixed.bucket_by_rate(rates)
    assert buckets.rates == [32, 48, 64]
    pairs = [make_bank(40 + b, len(m), H, I, n) for b, (m, n) in enumerate(zip(buckets.members, buckets.rates))]
    banks, obanks = [p[0] for p in pairs], [p[1] for p in pairs]
    for rows in (2, 48, 300):  # sub-banks see decode-row and prefill-row batches
        inds, scores = synth.routing(400 + rows, rows, E, topk)
        x16 = synth.activations(401 + rows, rows, H)
        y = mixed.mixed_rate_moe(dev(x16), banks, buckets, dev(inds), dev(scores), t3.Decode.mul1)
        sample = sorted({0, 1, rows // 2, rows - 1})
        v = np.zeros((len(sample), topk, H), np.float32)
        for si, r in enumerate(sample):
            for k in range(topk):
                e = int(inds[r, k])
                b, loc = int(buckets.bank_of[e]), int(buckets.local_of[e])
                v[si, k] = ob.moe_rows(obanks[b], x16[r:r + 1].astype(np.float32), np.array([[loc]], np.int32),
                                       np.ones((1, 1), np.float32))[0]
        check_moe(host_f32(y)[sample], _slot_sum(v, scores[sample]), "f16", ("config 4 mixed", rows))
    assert t3.device_error() == 0


@pytest.mark.parametrize("k", [2, 4])
def test_config5_large_layer(k):
    H, I, E, topk, n = 7168, 2048, 12, 8, 16 * k
    bank, obank = make_bank(50 + k, E, H, I, n)
    sbank, sobank = make_bank(60 + k, 1, H, I, n)
    for rows in (1, 4, 40):
        inds, scores = synth.routing(500 + rows, rows, E, topk, kind="sigmoid")
        x16 = synth.activations(501 + rows, rows, H)
        gate = (1.0 / (1.0 + np.exp(-np.random.default_rng(502 + rows).standard_normal((rows, 1))))).astype(np.float32)
        x = dev(x16).view(1, rows, H)
        zero = dev(np.zeros((rows, 1), np.int32)).view(1, rows, 1)
        shared = t3.moe(x, sbank, zero, dev(gate).view(1, rows, 1))
        y = t3.moe_with_shared(x, bank, dev(inds).view(1, rows, topk), dev(scores).view(1, rows, topk), t3.Decode.mul1, shared)
        sample = sorted({0, rows // 2, rows - 1})
        xs = x16[sample].astype(np.float32)
        half = lambda a: a.astype(np.float16).astype(np.float32)
        routed = ob.moe_rows(obank, xs, inds[sample], scores[sample])
        sh = ob.moe_rows(sobank, xs, np.zeros((len(sample), 1), np.int32), gate[sample])
        ref = half(half(routed) + half(sh))  # one add in the activation dtype (src/root.zig:975-984)
        check_moe(host_f32(y).reshape(rows, H)[sample], ref, "f16", ("config 5", k, rows), terms=1.5)
    assert t3.device_error() == 0


# name, in, out: the MLA-style attention projections, K = 4 (kv_a's 576 outputs padded to 640, a multiple of 128)
TRUNK = [("q_a", 7168, 1536), ("q_b", 1536, 24576), ("kv_a", 7168, 640), ("kv_b", 512, 32768), ("o", 16384, 7168)]


@pytest.mark.parametrize("proj", TRUNK)
def test_config5_trunk(proj):
    name, in_dim, out_dim = proj
    trellis, suh, svh = synth.linear(70 + in_dim % 97, in_dim, out_dim, 64)
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, 64, t3.MUL1, 16)
    t, a, b = dev(trellis), dev(suh), dev(svh)
    for rows in (1, 32, 200):
        x16 = synth.activations(71 + rows, rows, in_dim)
        y = t3.linear(dev(x16), t, a, b)
        sample = sorted({0, rows // 2, rows - 1})
        ref = ob.linear_rows_what(x16[sample].astype(np.float32), what, suh, svh, in_dim, out_dim)
        check(host_f32(y)[sample], ref, "f16", (name, rows))
    assert t3.device_error() == 0
