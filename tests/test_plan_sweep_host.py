"""Launch arithmetic of the decode-row kernels over a grid of shapes, rates and row counts, on the host: what a launch
needs to be a valid one (cluster, shared memory, grid) checked from the plan alone. No GPU is touched.

The reference plans its launches from the shape as well (src/hip/plan.zig, src/core/partition.zig:1-80); the splits here
are this library's own, so the properties are the ones any split must have.
"""
import itertools
import re

import pytest

import turboexl3_b200 as t3
from turboexl3_b200.api import lib

DIMS = [128, 256, 384, 512, 1536, 2048, 4096, 6144, 7168, 8192, 16384, 24576, 32768]
RATES = [16, 32, 48, 64, 80, 96, 112, 128, 20, 36, 100]   # halfwords a tile: the eight with kernels of their own, three without
ROWS = [1, 2, 7, 8, 9, 12, 16, 17, 31, 32]
SMEM_LIMIT = 200 * 1024   # what the library admits a CTA (the hardware's 227 KB less a reserve)
CLUSTER_MAX = 16          # the non-portable cluster size the kernels opt into


def _row_cap(rows):
    return 8 if rows <= 8 else (16 if rows <= 16 else 32)


@pytest.mark.parametrize("codebook", [t3.MUL1, t3.MCG])
def test_dense_plans_are_launchable(codebook):
    dec = t3.Decode(codebook)
    name = "mul1" if codebook == t3.MUL1 else "mcg"
    seen_global = seen_cluster = 0
    for (i, o), n, rows in itertools.product(itertools.product(DIMS, DIMS), RATES, ROWS):
        plan = t3.plan_linear(rows, i, o, n, dec)
        gemv = plan[-1]
        own = n if n % 16 == 0 else 0
        assert gemv["symbol"] == f"t3_dense_gemv_{name}_n{own}_r{_row_cap(rows)}", (i, o, n, rows)
        assert gemv["block"] == 544 and gemv["group"] == "dense"
        gx, gy, gz = gemv["grid"]
        assert gy == o // 128 and gz == 1 and 1 <= gx <= i // 128, (i, o, n, rows, gemv)  # a K slice holds a block at least
        assert 0 < gemv["shared"] <= SMEM_LIMIT, (i, o, n, rows, gemv)
        assert 1 <= gemv["cluster"] <= CLUSTER_MAX and gx % gemv["cluster"] == 0
        ws = lib().t3_linear_workspace_bytes(rows, i, o, n)
        if gemv["cluster"] == 1 and gx > 1:
            # slices that meet in global memory: the call asked for a workspace that holds every slice's partial sums
            assert ws >= gy * gx * rows * 128 * 4 + gy * 4, (i, o, n, rows, ws)
            seen_global += 1
        else:
            assert gx == gemv["cluster"]  # one cluster a 128-output block
            seen_cluster += 1
        if len(plan) == 2:
            prep = plan[0]
            assert prep["symbol"] == "t3_dense_prep" and prep["block"] == 128 and prep["cluster"] == 1
            assert prep["grid"] == ((rows * (i // 128) + 3) // 4, 1, 1)
            assert ws >= rows * i * 2  # the prepared rows (f16)
        else:
            assert len(plan) == 1
    assert seen_global > 0 and seen_cluster > 0
    for i, o in [(2048, 2048), (2048, 6144), (6144, 2048), (1536, 24576), (512, 32768)]:
        assert lib().t3_linear_workspace_bytes(1, i, o, 64) == 0  # one row of a trunk-sized linear runs without a workspace


def test_routed_plans_are_launchable():
    geoms = [(8, 128, 128), (10, 512, 2048), (64, 2048, 512), (128, 2048, 768), (256, 7168, 2048), (32, 4096, 1536), (16, 1024, 4096)]
    for (experts, hidden, inter), n, rows, topk in itertools.product(geoms, [16, 48, 64, 128, 36], [1, 3, 8, 16, 32], [1, 2, 8, 10]):
        if topk > experts:
            continue
        chain = t3.plan_moe(rows, topk, experts, hidden, inter, n)
        slots = rows * topk
        assert len(chain) == (2 if topk == 1 else 3), (experts, hidden, inter, n, rows, topk)
        gu, down = chain[0], chain[1]
        assert re.fullmatch(r"t3_dec_gate_up_mul1_n\d+_r(8|16|32)", gu["symbol"]) and re.fullmatch(r"t3_dec_down_mul1_n\d+_r(8|16|32)", down["symbol"])
        for l, blocks, k_blocks in ((gu, inter // 128, hidden // 128), (down, hidden // 128, inter // 128)):
            gx, gy, gz = l["grid"]
            assert (gy, gz) == (blocks, slots) and l["group"] == "decode" and l["block"] == 544
            assert gx == l["cluster"] and 1 <= l["cluster"] <= CLUSTER_MAX
            assert 0 < l["shared"] <= SMEM_LIMIT, (experts, hidden, inter, n, rows, topk, l)
        assert gu["cluster"] % 2 == 0 and gu["cluster"] // 2 <= hidden // 128  # gate and up side by side, a slice a block at least
        assert down["cluster"] <= inter // 128
        if topk > 1:
            merge = chain[2]
            assert merge["symbol"] == "t3_dec_merge" and merge["cluster"] == 1 and merge["shared"] < 48 * 1024


def test_plan_refusals_are_the_calls():
    for rows, i, o, n in [(0, 2048, 2048, 64), (1, 2048, 2040, 64), (1, 100, 2048, 64), (1, 2048, 2048, 14), (1, 2048, 2048, 130)]:
        with pytest.raises(t3.Exl3Error):
            t3.plan_linear(rows, i, o, n)
    with pytest.raises(t3.Exl3Error, match="BadExl3Shape"):
        t3.plan_moe(4, 33, 64, 512, 2048, 48)  # more slots a row than the merge takes (32)
    with pytest.raises(t3.Exl3Error, match="BadExl3Shape"):
        t3.plan_moe(4, 2, 10, 500, 2048, 48)  # hidden is not whole 128-blocks
    with pytest.raises(t3.Exl3Error, match="Exl3EngineNotImplemented"):
        t3.plan_moe(33, 2, 10, 512, 2048, 48)  # prefill rows: the plan covers the decode-row kernels


def test_prefill_workspace_holds_the_prepared_rows_and_a_bounded_slab():
    """Past 32 rows the workspace is the prepared rows (f16) plus, for calls of up to 512 rows that are cut into K slices, a slab
    of partial sums: a whole number of 64 KB tiles (128 x 128 f32 a slice a row tile), never more than two CTAs a
    multiprocessor's worth; nothing past 512 rows; and the same answer for every rate (the slab follows in and out alone)."""
    L = lib()
    up256 = lambda v: (v + 255) & ~255
    for i, o in itertools.product(DIMS, DIMS):
        for rows in (33, 128, 129, 256, 257, 512, 513, 4096):
            ws = L.t3_linear_workspace_bytes(rows, i, o, 64)
            xp = up256(rows * i * 2)
            assert ws >= xp, (i, o, rows)
            assert ws == L.t3_linear_workspace_bytes(rows, i, o, 36)
            if rows > 512:
                assert ws == xp, (i, o, rows)
                continue
            extra = ws - xp
            if extra:
                mtiles, ncol = (rows + 127) // 128, o // 128
                counters = up256(mtiles * ncol * 4)
                slab = extra - counters
                assert slab > 0 and slab % (mtiles * ncol * 65536) == 0, (i, o, rows, extra)
                slices = slab // (mtiles * ncol * 65536)
                assert 2 <= slices <= 8 and slices * 4 <= i // 64, (i, o, rows, slices)
                assert mtiles * ncol * slices <= 2 * 148, (i, o, rows, slices)  # two CTAs a multiprocessor at most (148 of them)
        # within an arm the slice count does not depend on the rows
        for lo, hi in ((33, 256), (257, 512)):
            per_tile = set()
            for rows in (lo, (lo + hi) // 2, hi):
                extra = L.t3_linear_workspace_bytes(rows, i, o, 64) - up256(rows * i * 2)
                mtiles, ncol = (rows + 127) // 128, o // 128
                per_tile.add((extra - up256(mtiles * ncol * 4)) // (mtiles * ncol * 65536) if extra else 1)
            assert len(per_tile) == 1, (i, o, lo, hi, per_tile)
