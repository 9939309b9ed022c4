"""The oracle against every known-answer value and identity the reference's own CPU tests hold for this path
(src/core/format.zig:427-571, src/core/lane.zig:244-254, src/core/ref.zig:284-306)."""
import numpy as np
import pytest

from oracle import binding as ob

L = ob.lib()


def test_mul1_pins():  # format.zig:427-431
    assert L.t3o_decode_mul1(0) == 49896
    assert L.t3o_decode_mul1(1) == 14625
    assert L.t3o_decode_mul1(7) == 47511


def test_multipliers():  # format.zig:433-439
    assert L.t3o_multiplier(ob.MUL1) == 0x83DCD12D
    assert L.t3o_multiplier(ob.MCG) == 0xCBAC1FED


def test_mcg_zero():  # format.zig:441-445
    want = L.t3o_f32_to_f16_bits(L.t3o_f16_bits_to_f32(0x3B60) + L.t3o_f16_bits_to_f32(0x3B60))
    assert L.t3o_decode_mcg(0) == want == 16224


def test_windows():  # format.zig:447-457
    assert L.t3o_window_mask(16) == 0xFFFF
    assert L.t3o_window_mask(12) == 0x0FFF
    assert L.t3o_window_mask(8) == 0xFF
    assert L.t3o_window_mask(15) == 0x7FFF
    assert L.t3o_window_mask(7) == -1
    assert L.t3o_window_mask(17) == -1


def test_rates():  # format.zig:459-478
    for bad in (15, 130, 49):
        assert not L.t3o_rate_admitted(bad)
    for n in range(16, 130, 2):
        assert L.t3o_rate_admitted(n)
        assert L.t3o_bit_end(n, 255) == 16 * n
        assert sum(L.t3o_fresh_bits(n, t) for t in range(256)) == 16 * n
    assert L.t3o_bit_end(64, 0) == 4
    assert L.t3o_bit_end(80, 15) == 80
    assert L.t3o_bit_end(36, 0) == 2
    assert L.t3o_bit_end(36, 3) == 9


def test_unpack_matches_definition_every_rate():  # format.zig:480-492
    rng = np.random.default_rng(0xE7135EED)
    for n in range(16, 130, 2):
        words = rng.integers(0, 65536, n, dtype=np.uint16)
        assert np.array_equal(ob.unpack_tile(words, n), ob.codewords_by_definition(words, n)), n


def test_packer_round_trip():  # format.zig:494-510
    rng = np.random.default_rng(0x5EED5EED)
    for k in range(1, 9):
        sym = rng.integers(0, 1 << k, 256, dtype=np.uint16)
        words = ob.pack_symbols(sym, k)
        got = ob.unpack_tile(words, 16 * k)
        assert np.array_equal(got & ((1 << k) - 1), sym), k


def test_perm():  # format.zig:512-523
    p = ob.tensor_core_perm()
    assert sorted(p.tolist()) == list(range(256))
    assert (p[0], p[1], p[4]) == (0, 16, 8)


def test_hadamard_involution():  # format.zig:525-532
    v = np.array([(i % 17) - 8.0 for i in range(128)], np.float32)
    w = ob.hadamard128(ob.hadamard128(v))
    assert np.max(np.abs(v - w)) < 1e-4
    assert L.t3o_had_scale() == float(np.float32(0.08838834764831845))


def test_project_vs_public_weight():  # format.zig:534-571
    rng = np.random.default_rng(0x7E57)
    in_f = out_f = 128
    n = 64
    trellis = rng.integers(0, 65536, (in_f // 16) * (out_f // 16) * n, dtype=np.uint16)
    suh = (0.5 + rng.random(in_f, dtype=np.float32)).astype(np.float16)
    svh = (0.5 + rng.random(out_f, dtype=np.float32)).astype(np.float16)
    pub = ob.reconstruct_public(trellis, suh, svh, in_f, out_f, n, ob.MUL1).view(np.float16).astype(np.float32)
    x = rng.random(in_f, dtype=np.float32) - 0.5
    y = ob.project(x, trellis, suh, svh, in_f, out_f, n, ob.MUL1)
    xr = x.astype(np.float16).astype(np.float32)
    acc = np.zeros(out_f, np.float32)
    for r in range(in_f):
        acc += xr[r] * pub[r]
    assert np.max(np.abs(acc)) > 0
    assert np.max(np.abs(acc - y)) <= 0.02 * np.max(np.abs(acc))


def test_mul1_integer_route():  # lane.zig:244-254: t -> f16(0x6400 + t) -> fma is decodeMul1
    for cw in (0, 1, 7, 0x1234, 0xFFFF):
        t = L.t3o_mul1_t(cw)
        assert 0 <= t <= 1020
        h = np.array([0x6400 + t], np.uint16).view(np.float16).astype(np.float64)[0]
        a = np.array([0x1EEE], np.uint16).view(np.float16).astype(np.float64)[0]
        b = np.array([0xC931], np.uint16).view(np.float16).astype(np.float64)[0]
        assert np.float16(h * a + b).view(np.uint16) == L.t3o_decode_mul1(cw)


def test_mul1_single_rounding_is_exact_for_every_t():
    """h*A + B needs at most 20 significant bits for every byte sum t, so the reference's f32 fma is exact and one
    rounding to f16 (what a half-precision fma does) gives decodeMul1's bits: the CUDA kernels rely on this."""
    a = float(np.array([0x1EEE], np.uint16).view(np.float16)[0])
    b = float(np.array([0xC931], np.uint16).view(np.float16)[0])
    seen = {}
    for cw in range(65536):
        seen.setdefault(L.t3o_mul1_t(cw), cw)
    assert len(seen) > 900
    for t, cw in seen.items():
        exact = (1024.0 + t) * a + b  # exact in f64
        assert float(np.float32(exact)) == exact
        assert np.float16(exact).view(np.uint16) == L.t3o_decode_mul1(cw)


def test_mcg_half_add_is_exact_for_every_codeword():
    """MCG's two halves sum exactly in f32, so a single half-precision add gives decodeMcg's bits."""
    cws = np.arange(65536, dtype=np.uint64)
    pair = 0x3B603B60 ^ ((cws * 0xCBAC1FED) & 0xFFFFFFFF & 0x8FFF8FFF)
    lo = (pair & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
    hi = (pair >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
    want = ob.decode_table(ob.MCG)
    assert np.array_equal((lo + hi).astype(np.float16).view(np.uint16), want)


def _synth_bank(rng, experts, hidden, inter, n):
    gu = experts * (hidden // 16) * (inter // 16) * n
    f16 = lambda a: a.astype(np.float16)
    return ob.Bank(
        experts, hidden, inter, n,
        rng.integers(0, 65536, gu, dtype=np.uint16), f16(0.5 + rng.random(experts * hidden)),
        f16((0.5 + rng.random(experts * inter)) / np.sqrt(hidden)),
        rng.integers(0, 65536, gu, dtype=np.uint16), f16(0.5 + rng.random(experts * hidden)),
        f16((0.5 + rng.random(experts * inter)) / np.sqrt(hidden)),
        rng.integers(0, 65536, gu, dtype=np.uint16), f16(0.5 + rng.random(experts * inter)),
        f16((0.5 + rng.random(experts * hidden)) / np.sqrt(inter)))


def test_moe_row_finite_and_slot_order():  # ref.zig:284-306
    rng = np.random.default_rng(0x5EED)
    bank = _synth_bank(rng, 4, 256, 128, 64)
    x = rng.standard_normal(256).astype(np.float32)
    y = ob.moe_rows(bank, x, [1, 3], [0.7, 0.3], threads=1)[0]
    assert np.all(np.isfinite(y))
    rms = float(np.sqrt(np.mean(y.astype(np.float64) ** 2)))
    assert 1e-3 < rms < 100.0
    y2 = ob.moe_rows(bank, x, [3, 1], [0.3, 0.7], threads=1)[0]
    assert ob.compare(y2, y)["max_ratio"] < 1e-5


def test_threaded_drivers_equal_single_thread():
    rng = np.random.default_rng(11)
    in_f, out_f, n = 256, 384, 48
    trellis = rng.integers(0, 65536, (in_f // 16) * (out_f // 16) * n, dtype=np.uint16)
    suh = np.where(rng.random(in_f) < 0.5, -1, 1).astype(np.float16)
    svh = np.where(rng.random(out_f) < 0.5, -1, 1).astype(np.float16)
    x = rng.standard_normal((3, in_f)).astype(np.float32)
    y1 = ob.linear_rows(x, trellis, suh, svh, in_f, out_f, n, ob.MCG, 12, threads=1)
    y4 = ob.linear_rows(x, trellis, suh, svh, in_f, out_f, n, ob.MCG, 12, threads=4)
    assert np.array_equal(y1.view(np.uint32), y4.view(np.uint32))
    what = ob.reconstruct_inner(trellis, in_f, out_f, n, ob.MCG, 12)
    yw = ob.linear_rows_what(x, what, suh, svh, in_f, out_f, threads=3)
    assert np.array_equal(y1.view(np.uint32), yw.view(np.uint32))
    for r in range(3):
        assert np.array_equal(ob.project(x[r], trellis, suh, svh, in_f, out_f, n, ob.MCG, 12), y1[r])


@pytest.mark.parametrize("limit,clamp_at", [(0.0, 0), (1.0, 0), (1.0, 1)])
def test_swiglu_clamps(limit, clamp_at):  # ref.zig:124-140
    f = L.t3o_swiglu_clamped_out if clamp_at else L.t3o_swiglu_clamped
    g, u = 3.0, -5.0
    silu = lambda v: v / (1.0 + np.exp(-v))
    if limit == 0:
        want = silu(g) * u
    elif clamp_at == 0:
        want = silu(min(g, limit)) * max(-limit, min(u, limit))
    else:
        want = min(silu(g), limit) * max(-limit, min(u, limit))
    assert abs(f(g, u, limit) - want) < 1e-6
