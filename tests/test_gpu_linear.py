"""The dense EXL3 linear against the oracle's format.project, at the shapes and row counts of the reference's own GPU
tests (src/hip_tests.zig:294-347, src/core/gpu_test.zig:384-398) and of the benchmark configs 1 and 2.

Bars (gpu_util.check): the reference's own `ref.compare` max|err|/rms <= 5e-3 for f32/f16 activations and <= 2.5e-2
for bf16 (src/core/gpu_test.zig:46,438,446), plus compareRounded(half ulp of the output dtype) <= 3e-3."""
import numpy as np
import pytest
import torch

import turboexl3_b200 as t3
from oracle import binding as ob
from turboexl3_b200 import synth

from gpu_util import bits16, check, dev, host_f32, x_as

pytestmark = pytest.mark.gpu


def run_case(in_dim, out_dim, n, codebook, window, dt, rows, seed, scaled=True):
    trellis, suh, svh = synth.linear(seed, in_dim, out_dim, n, scaled=scaled)
    x16 = synth.activations(seed + 1, rows, in_dim)
    x = x_as(x16, dt)
    dec = t3.Decode(codebook, window)
    y = t3.linear(x, dev(trellis), dev(suh), dev(svh), dec)
    assert y.shape == (rows, out_dim) and y.dtype == x.dtype
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, codebook, window)
    ref = ob.linear_rows_what(host_f32(x), what, suh, svh, in_dim, out_dim)
    assert np.all(np.isfinite(ref))
    return host_f32(y), ref, y


# (in, out, n, codebook, window, dtype): src/hip_tests.zig:294-347
HIP_CASES = [
    (512, 256, 64, t3.MCG, 16, "f32"), (512, 256, 64, t3.MUL1, 16, "f32"), (512, 384, 32, t3.MCG, 16, "f16"),
    (512, 256, 48, t3.MUL1, 16, "f16"), (512, 256, 36, t3.MCG, 16, "f32"), (512, 256, 128, t3.MCG, 12, "f16"),
    (2560, 640, 80, t3.MUL1, 16, "bf16"), (4096, 2048, 64, t3.MCG, 16, "bf16"),
]


@pytest.mark.parametrize("case", HIP_CASES)
def test_reference_gemv_cases(case):
    in_dim, out_dim, n, cb, w, dt = case
    for rows in (1, 2, 3, 4, 5, 6, 7, 8, 9, 11, 16, 17, 31, 32):
        got, ref, _ = run_case(in_dim, out_dim, n, cb, w, dt, rows, seed=in_dim + n + rows)
        check(got, ref, dt, (case, rows))
    assert t3.device_error() == 0


def test_config1_single_linear():
    """Benchmark config 1: 4096 x 4096, K = 4, seed 0, +-1 signs, one f16 row."""
    got, ref, _ = run_case(4096, 4096, 64, t3.MUL1, 16, "f16", 1, seed=0, scaled=False)
    check(got, ref, "f16", "config 1")


@pytest.mark.parametrize("shape", [(2048, 2048), (2048, 6144), (6144, 2048)])
@pytest.mark.parametrize("k", [1, 2, 3, 4, 5, 6, 8])
def test_config2_sweep_decode_rows(shape, k):
    """Benchmark config 2 at the in-register rows {1, 8, 17, 32}, +-1 signs."""
    in_dim, out_dim = shape
    for rows in (1, 8, 17, 32):
        got, ref, _ = run_case(in_dim, out_dim, 16 * k, t3.MUL1, 16, "f16", rows, seed=7 * k + rows, scaled=False)
        check(got, ref, "f16", (shape, k, rows))
    assert t3.device_error() == 0


# (in, out, n, codebook, window, dtype): the reference's GEMM cases (src/hip_tests.zig:839-881, src/core/gpu_test.zig:384-398)
GEMM_CASES = [
    (512, 256, 64, t3.MCG, 16, "f32"), (512, 256, 64, t3.MUL1, 16, "f16"), (512, 384, 36, t3.MUL1, 12, "f16"),
    (2560, 640, 80, t3.MUL1, 16, "bf16"), (640, 2560, 112, t3.MUL1, 16, "f16"), (2560, 512, 96, t3.MCG, 16, "f16"),
]


@pytest.mark.parametrize("case", GEMM_CASES)
def test_reference_gemm_cases(case):
    """rows > 32: prepare -> tcgen05 GEMM with the trellis decoded in its weight loader -> finish."""
    in_dim, out_dim, n, cb, w, dt = case
    for rows in (33, 40, 129, 200, 256, 257, 600):
        got, ref, _ = run_case(in_dim, out_dim, n, cb, w, dt, rows, seed=in_dim + rows)
        check(got, ref, dt, (case, rows))
    assert t3.device_error() == 0


def test_config2_sweep_gemm_rows():
    """Benchmark config 2 at the GEMM rows {33, 512, 4096}: every K at 2048x2048, K = 4 at the two wide shapes; +-1 signs."""
    cases = [((2048, 2048), k) for k in (1, 2, 3, 4, 5, 6, 8)] + [((2048, 6144), 4), ((6144, 2048), 4)]
    for (in_dim, out_dim), k in cases:
        for rows in (33, 512, 4096):
            if rows == 4096 and (in_dim, out_dim) != (2048, 2048):
                continue  # the oracle is the slow side
            got, ref, _ = run_case(in_dim, out_dim, 16 * k, t3.MUL1, 16, "f16", rows, seed=11 * k + rows, scaled=False)
            check(got, ref, "f16", ((in_dim, out_dim), k, rows))
    assert t3.device_error() == 0


def test_gemm_first_rows_are_byte_stable():
    """The first 17 rows' bytes are the same in a 40-row and a 200-row call (src/hip_tests.zig:870-880)."""
    trellis, suh, svh = synth.linear(51, 512, 256, 64, scaled=True)
    t, a, b = dev(trellis), dev(suh), dev(svh)
    x = dev(synth.activations(52, 200, 512))
    y200 = bits16(t3.linear(x, t, a, b))
    y40 = bits16(t3.linear(x[:40].contiguous(), t, a, b))
    assert np.array_equal(y200[:17], y40[:17])


def test_a_row_alone_equals_the_row_in_a_batch():
    """A row's bytes do not depend on its neighbours (src/hip_tests.zig:330-345, src/core/gpu_test.zig:708)."""
    in_dim, out_dim, n = 2560, 640, 80
    trellis, suh, svh = synth.linear(3, in_dim, out_dim, n, scaled=True)
    t, a, b = dev(trellis), dev(suh), dev(svh)
    for rows in (7, 16, 32):
        x = dev(synth.activations(40 + rows, rows, in_dim))
        full = bits16(t3.linear(x, t, a, b))
        for r in (0, rows // 2, rows - 1):
            alone = bits16(t3.linear(x[r:r + 1].contiguous(), t, a, b))
            assert np.array_equal(alone[0], full[r]), (rows, r)


def test_same_call_twice_same_bytes():
    trellis, suh, svh = synth.linear(9, 2048, 2048, 48)
    x = dev(synth.activations(10, 5, 2048))
    t, a, b = dev(trellis), dev(suh), dev(svh)
    assert np.array_equal(bits16(t3.linear(x, t, a, b)), bits16(t3.linear(x, t, a, b)))


def test_leading_dims_are_rows():
    trellis, suh, svh = synth.linear(12, 256, 128, 64)
    x = dev(synth.activations(13, 6, 256))
    t, a, b = dev(trellis), dev(suh), dev(svh)
    y2 = t3.linear(x, t, a, b)
    y3 = t3.linear(x.view(2, 3, 256), t, a, b)
    assert y3.shape == (2, 3, 128)
    assert np.array_equal(bits16(y2), bits16(y3).reshape(6, 128))


def test_split_choices_agree_within_rounding():
    """The cluster's K split only changes f32 summation order."""
    trellis, suh, svh = synth.linear(21, 2048, 512, 64, scaled=True)
    x = dev(synth.activations(22, 4, 2048))
    t, a, b = dev(trellis), dev(suh), dev(svh)
    outs = []
    try:
        for split in (1, 2, 3, 4, 5, 7, 8, 16):
            t3.configure(dense_split=split)
            outs.append(host_f32(t3.linear(x, t, a, b)))
    finally:
        t3.configure()
    for o in outs[1:]:
        assert ob.compare(o, outs[0], 2.0 ** -11)["max_ratio"] <= 3e-3


def test_small_ring_recycles_stages():
    """A ring far smaller than the slab forces every stage to be reused many times."""
    trellis, suh, svh = synth.linear(31, 4096, 256, 128, scaled=True)
    x = dev(synth.activations(32, 3, 4096))
    t, a, b = dev(trellis), dev(suh), dev(svh)
    base = bits16(t3.linear(x, t, a, b))
    try:
        t3.configure(ring_bytes=8192, dense_split=1)
        small = host_f32(t3.linear(x, t, a, b))
        t3.configure(ring_bytes=8192, dense_split=8)
        small8 = bits16(t3.linear(x, t, a, b))
    finally:
        t3.configure()
    assert np.array_equal(small8, base)
    what = ob.reconstruct_inner(trellis, 4096, 256, 128, ob.MUL1)
    ref = ob.linear_rows_what(host_f32(x), what, suh, svh, 4096, 256)
    check(small, ref, "f16", "ring of one stage")
    assert t3.device_error() == 0


@pytest.mark.parametrize("n,cb", [(48, t3.MUL1), (128, t3.MCG), (36, t3.MUL1)])
def test_gemm_512_row_tiles(n, cb):
    """Calls large enough to fill the GPU with 512-row tiles (four accumulators a decoded tile): a ragged last tile, rows
    sampled in every quarter of a tile, and the same bytes as the 256-row-tile path gives the leading rows."""
    in_dim, out_dim, rows = 512, 2560, 4100
    trellis, suh, svh = synth.linear(600 + n, in_dim, out_dim, n, scaled=True)
    x16 = synth.activations(601 + n, rows, in_dim)
    dec = t3.Decode(cb, 16)
    t, a, b, x = dev(trellis), dev(suh), dev(svh), dev(x16)
    y = t3.linear(x, t, a, b, dec)
    sample = [0, 127, 128, 255, 256, 383, 384, 511, 512, 1000, 2047, 2048, 3583, 4095, 4096, 4099]
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, cb, 16)
    ref = ob.linear_rows_what(x16[sample].astype(np.float32), what, suh, svh, in_dim, out_dim)
    check(host_f32(y)[sample], ref, "f16", ("512-row tiles", n))
    small = t3.linear(x[:700].contiguous(), t, a, b, dec)  # 256-row tiles: the same K order a row
    assert np.array_equal(bits16(y[:700]), bits16(small))
    assert t3.device_error() == 0


def test_engines_held_counts_geometries_and_release_empties_them():
    t3.release_engines()
    trellis, suh, svh = synth.linear(700, 256, 128, 32, scaled=True)
    t, a, b = dev(trellis), dev(suh), dev(svh)
    for rows in (1, 5, 40, 50):
        t3.linear(dev(synth.activations(701, rows, 256)), t, a, b)
    assert t3.engines_held() == {"decode": 0, "dense": 1, "prefill": 1}
    t3.release_engines()
    assert t3.engines_held() == {"decode": 0, "dense": 0, "prefill": 0}


@pytest.mark.parametrize("case", [(512, 2560, 48, t3.MUL1), (640, 256, 128, t3.MCG), (2048, 2048, 36, t3.MUL1)])
def test_resident_trunk_gives_the_per_call_bytes(case):
    """src/core/dense.zig:1323-1530: a kept W_hat is the per-call one bit for bit, and so is every output; decode rows never
    touch it."""
    from turboexl3_b200.resident import ResidentTable
    in_dim, out_dim, n, cb = case
    trellis, suh, svh = synth.linear(800 + n, in_dim, out_dim, n, scaled=True)
    dec = t3.Decode(cb, 16)
    t, a, b = dev(trellis), dev(suh), dev(svh)
    w_t = t3.resident_build(t, dec)
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, cb, 16)
    assert np.array_equal(bits16(w_t), np.ascontiguousarray(what.T).view(np.uint16))
    table = ResidentTable()
    table.arm([t])
    assert table.pending() == in_dim * out_dim * 2 and not table.keeps(t)
    for rows in (1, 33, 300, 4100):
        x = dev(synth.activations(801 + rows, rows, in_dim))
        assert np.array_equal(bits16(table.linear(x, t, a, b, dec)), bits16(t3.linear(x, t, a, b, dec))), rows
        assert table.keeps(t) == (rows > 32)
    assert table.pending() == 0 and table.stats()["kept_bytes"] == in_dim * out_dim * 2
    table.release()
    assert table.stats() == {"admitted": 0, "kept": 0, "kept_bytes": 0}
    assert t3.device_error() == 0


def test_scales_that_are_not_signs():
    """suh / svh with magnitudes in [0.5, 1.5] (the reference's synthetic scales, src/core/ref.zig:66-73): x * suh is then not
    an f16 value, and the prepare's tensor-core Hadamard takes its two-part path."""
    rng = np.random.default_rng(900)
    in_dim, out_dim, n = 1024, 384, 64
    trellis, suh, svh = synth.linear(901, in_dim, out_dim, n)
    suh = (suh.astype(np.float32) * rng.uniform(0.5, 1.5, in_dim)).astype(np.float16)
    svh = (svh.astype(np.float32) * rng.uniform(0.5, 1.5, out_dim) / 32.0).astype(np.float16)
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, t3.MUL1, 16)
    t, a, b = dev(trellis), dev(suh), dev(svh)
    for rows, dt in ((1, "f16"), (32, "f16"), (33, "f16"), (300, "f32"), (600, "bf16")):
        x = x_as(synth.activations(902 + rows, rows, in_dim), dt)
        y = t3.linear(x, t, a, b)
        ref = ob.linear_rows_what(host_f32(x), what, suh, svh, in_dim, out_dim)
        check(host_f32(y), ref, dt, ("general scales", rows, dt))
    assert t3.device_error() == 0


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_lives_on():
    """A copy that never lands must not hang the GPU: the kernels' waits are bounded, the one that gives up sets a bit in
    the device error word, and the next call runs as usual."""
    assert t3.device_error() == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert t3.lib().t3_selftest_wait_runs_out(stream) == 0
    bits = t3.device_error()  # synchronises; clears
    assert bits == 1, bits
    assert t3.device_error() == 0
    trellis, suh, svh = synth.linear(3, 256, 256, 32, scaled=True)
    x = synth.activations(4, 1, 256)
    y = t3.linear(dev(x), dev(trellis), dev(suh), dev(svh))
    ref = ob.linear_rows(x.astype(np.float32), trellis, suh, svh, 256, 256, 32, ob.MUL1)
    assert ob.compare(host_f32(y), ref)["max_ratio"] <= 5e-3
    assert t3.device_error() == 0


def test_timing_probes_run_in_the_served_kernels_place():
    """The dense GEMV's probes (hash skipped, window extraction skipped, stream only) launch, finish and set no error;
    their outputs are not the linear's, and serving comes back when the probe is switched off."""
    trellis, suh, svh = synth.linear(5, 1024, 512, 64, scaled=True)
    x = dev(synth.activations(6, 3, 1024))
    args = (x, dev(trellis), dev(suh), dev(svh))
    served = t3.linear(*args)
    try:
        for mode in (1, 2, 3):
            t3.configure(probe=mode)
            y = t3.linear(*args)
            assert y.shape == served.shape
            assert t3.device_error() == 0
            with pytest.raises(t3.Exl3Error, match="Exl3EngineNotImplemented"):
                t3.linear(dev(synth.activations(6, 9, 1024)), *args[1:])
        with pytest.raises(t3.Exl3Error, match="InvalidTurboexl3Config"):
            t3.configure(probe=4)
    finally:
        t3.configure()
    assert torch.equal(t3.linear(*args), served)


def test_large_linear_global_exchange_matches_the_cluster_kernel_within_bars():
    """Linears of 24 MB of codes and up, given their workspace, let the K slices' sums meet in global memory (any slice
    count, CTAs placed one by one); without the workspace the cluster kernel runs. Different K partitions, so not the same
    bytes, but each within the dense bars of the oracle; the same call twice gives the same bytes."""
    in_dim, out_dim, n = 16384, 7168, 32  # K2: 29 MB of codes
    L = t3.lib()
    assert L.t3_linear_workspace_bytes(1, in_dim, out_dim, n) > 0
    plan = t3.plan_linear(1, in_dim, out_dim, n)
    assert plan[-1]["cluster"] == 1 and plan[-1]["grid"][0] not in (1, 2, 4, 8, 16)
    rng = np.random.default_rng(5)
    trellis = rng.integers(0, 65536, size=(in_dim // 16, out_dim // 16, n), dtype=np.uint16)
    _, suh, svh = synth.linear(6, in_dim, 128, 16)
    svh = np.where(rng.random(out_dim) < 0.5, -1.0, 1.0).astype(np.float16)
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, ob.MUL1)
    for rows in (1, 7, 12, 32):  # 7: the rows rotated ahead as well; 12, 32: whichever exchange their prepared rows leave room for
        x = synth.activations(7, rows, in_dim)
        args = (dev(x), dev(trellis.view(np.int16)), dev(suh), dev(svh))
        y = t3.linear(*args)  # api.linear brings the workspace
        assert t3.last_kernel_symbol().startswith("t3_dense_gemv_mul1_n32")
        assert torch.equal(y, t3.linear(*args))
        yb = torch.empty_like(y)
        rc = L.t3_linear(args[0].data_ptr(), 1, rows, args[1].data_ptr(), args[2].data_ptr(), args[3].data_ptr(), in_dim, out_dim, n,
                         t3.Decode.mul1._c(), yb.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        ref = ob.linear_rows_what(x.astype(np.float32), what, suh, svh, in_dim, out_dim)
        for got in (y, yb):
            check(host_f32(got), ref, "f16", f"large_linear_rows{rows}")
    assert t3.device_error() == 0


@pytest.mark.parametrize("rows", [9, 16, 17, 32])
def test_rows_past_8_with_and_without_the_workspace_give_the_same_bytes(rows):
    """Past 8 rows the workspace is optional: with it the rows are rotated once by a launch of their own and the CTAs pull
    them by bulk copy, without it every CTA rotates its own copy. The same arithmetic on the same K slices: the same bytes."""
    in_dim, out_dim, n = 1024, 768, 48
    trellis, suh, svh = synth.linear(21, in_dim, out_dim, n, scaled=True)
    x = dev(synth.activations(22, rows, in_dim))
    args = (x, dev(trellis), dev(suh), dev(svh))
    L = t3.lib()
    assert L.t3_linear_workspace_bytes(rows, in_dim, out_dim, n) >= rows * in_dim * 2
    with_ws = t3.linear(*args)
    assert t3.launch_count() > 0
    without = torch.empty_like(with_ws)
    before = t3.launch_count()
    rc = L.t3_linear(x.data_ptr(), 1, rows, args[1].data_ptr(), args[2].data_ptr(), args[3].data_ptr(), in_dim, out_dim, n,
                     t3.Decode.mul1._c(), without.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and t3.launch_count() - before == 1  # one launch: no prepare of its own
    assert torch.equal(with_ws, without)
    assert t3.device_error() == 0


@pytest.mark.parametrize("case", [(6144, 2048, 64, t3.MUL1, 512), (2048, 6144, 64, t3.MUL1, 40), (2048, 2048, 36, t3.MCG, 130),
                                  (7168, 1536, 48, t3.MUL1, 400), (1536, 24576, 64, t3.MUL1, 200), (16384, 7168, 32, t3.MUL1, 64)])
def test_gemm_of_few_rows_cuts_k_into_slices(case):
    """Calls of 33..256 and of 257..512 rows are few tall CTAs, so K is cut into slices that meet in global memory (the tile's last arriver
    adds them in slice order). Within the dense bars of the oracle on sampled rows; the same call twice gives the same
    bytes; a row's bytes do not depend on the call's row count within an arm (src/hip_tests.zig:870-880 asks it of the first 17
    rows of 40- and 200-row calls)."""
    in_dim, out_dim, n, cb, rows = case
    trellis, suh, svh = synth.linear(1300 + rows, in_dim, out_dim, n, scaled=True)
    x16 = synth.activations(1301 + rows, rows, in_dim)
    dec = t3.Decode(cb, 16)
    t, a, b, x = dev(trellis), dev(suh), dev(svh), dev(x16)
    y = t3.linear(x, t, a, b, dec)
    sample = sorted({0, 1, 16, 31, 32, rows // 2, min(rows - 1, 127), min(rows - 1, 128), rows - 2, rows - 1})
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, cb, 16)
    ref = ob.linear_rows_what(x16[sample].astype(np.float32), what, suh, svh, in_dim, out_dim)
    check(host_f32(y)[sample], ref, "f16", ("K slices", case))
    assert np.array_equal(bits16(y), bits16(t3.linear(x, t, a, b, dec)))
    few = 33 if rows <= 256 else 257  # the fewest rows of the call's arm
    head = t3.linear(x[:few].contiguous(), t, a, b, dec)
    assert np.array_equal(bits16(y[:few]), bits16(head))
    assert t3.device_error() == 0

