"""Generates tests/golden/golden.npz from the pinned CPU oracle (oracle/t3_oracle.c).

The reference's own seeded fixtures cannot be replayed (they draw from Zig's PRNG and record no output values), and the
reference cannot run in this environment, so these vectors are ORACLE-generated regression fixtures: they freeze the
oracle's outputs once it passes every literal pin of the reference's CPU tests (tests/test_oracle_pins.py), and the CUDA
path is held to them on the GPU.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import binding as ob  # noqa: E402
from turboexl3_b200 import synth  # noqa: E402


def main() -> None:
    out = {}
    # one tile at every integer rate and three fractional ones: words in, 256 decoded f16 out (row-major), both codebooks
    rng = np.random.default_rng(20240229)
    for n in (16, 32, 48, 64, 80, 96, 112, 128, 36, 56, 104):
        words = rng.integers(0, 65536, n, dtype=np.uint16)
        out[f"tile_n{n}_words"] = words
        out[f"tile_n{n}_codewords"] = ob.unpack_tile(words, n)
        for cb, name in ((ob.MUL1, "mul1"), (ob.MCG, "mcg")):
            out[f"tile_n{n}_{name}_w16"] = ob.reconstruct_inner(np.tile(words, 64), 128, 128, n, cb, 16)[:16, :16].copy()
        out[f"tile_n{n}_mcg_w12"] = ob.reconstruct_inner(np.tile(words, 64), 128, 128, n, ob.MCG, 12)[:16, :16].copy()
    # a 256 x 384 linear at K = 3 (MUL1) and n = 40 (MCG, window 12): W_hat and three projected rows with their stages
    for tag, n, cb, w in (("lin_k3_mul1", 48, ob.MUL1, 16), ("lin_n40_mcg_w12", 40, ob.MCG, 12)):
        trellis, suh, svh = synth.linear(4242 + n, 256, 384, n, scaled=True)
        x = synth.activations(4243 + n, 3, 256)
        out[f"{tag}_trellis"], out[f"{tag}_suh"], out[f"{tag}_svh"], out[f"{tag}_x"] = trellis, suh, svh, x
        out[f"{tag}_what"] = ob.reconstruct_inner(trellis, 256, 384, n, cb, w)
        ys, xps, zs = [], [], []
        for r in range(3):
            y, xp, z = ob.project(x[r].astype(np.float32), trellis, suh, svh, 256, 384, n, cb, w, stages=True)
            ys.append(y), xps.append(xp), zs.append(z)
        out[f"{tag}_y"], out[f"{tag}_xp"], out[f"{tag}_z"] = np.stack(ys), np.stack(xps), np.stack(zs)
    # a routed layer: hidden 256, width 128, 6 experts, top-3, K = 4, two rows, with the per-slot outputs
    arrs = synth.bank(777, 6, 256, 128, 64)
    bank = ob.Bank(6, 256, 128, 64, *[arrs[k] for k in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh", "up_svh",
                                                          "down_t", "down_suh", "down_svh")])
    inds, scores = synth.routing(778, 2, 6, 3)
    x = synth.activations(779, 2, 256)
    y, per_slot = ob.moe_rows(bank, x.astype(np.float32), inds, scores, per_slot=True)
    for k, v in arrs.items():
        out[f"moe_{k}"] = v
    out["moe_inds"], out["moe_scores"], out["moe_x"], out["moe_y"], out["moe_per_slot"] = inds, scores, x, y, per_slot
    y_c, _ = ob.moe_rows(bank, x.astype(np.float32), inds, scores, limit=1.0, per_slot=True)
    out["moe_y_clamped_gate_in_1"] = y_c
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
