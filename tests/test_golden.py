"""Golden vectors (tests/golden/golden.npz, made by tests/golden/make_golden.py from the pinned oracle): the oracle must
keep reproducing them on the CPU, and the CUDA path is held to them on the GPU."""
import os

import numpy as np
import pytest

from oracle import binding as ob

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
RATES = (16, 32, 48, 64, 80, 96, 112, 128, 36, 56, 104)


def test_oracle_reproduces_tiles():
    for n in RATES:
        words = G[f"tile_n{n}_words"]
        assert np.array_equal(ob.unpack_tile(words, n), G[f"tile_n{n}_codewords"])
        for cb, name, w in ((ob.MUL1, "mul1", 16), (ob.MCG, "mcg", 16), (ob.MCG, "mcg", 12)):
            got = ob.reconstruct_inner(np.tile(words, 64), 128, 128, n, cb, w)[:16, :16]
            assert np.array_equal(got, G[f"tile_n{n}_{name}_w{w}"]), (n, name, w)


def test_oracle_reproduces_linears_and_layer():
    for tag, n, cb, w in (("lin_k3_mul1", 48, ob.MUL1, 16), ("lin_n40_mcg_w12", 40, ob.MCG, 12)):
        t, a, b, x = (G[f"{tag}_{k}"] for k in ("trellis", "suh", "svh", "x"))
        assert np.array_equal(ob.reconstruct_inner(t, 256, 384, n, cb, w), G[f"{tag}_what"])
        for r in range(3):
            y, xp, z = ob.project(x[r].astype(np.float32), t, a, b, 256, 384, n, cb, w, stages=True)
            assert np.array_equal(y, G[f"{tag}_y"][r]) and np.array_equal(xp, G[f"{tag}_xp"][r])
            assert np.array_equal(z, G[f"{tag}_z"][r])
    bank = ob.Bank(6, 256, 128, 64, *[G[f"moe_{k}"] for k in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh",
                                                                 "up_svh", "down_t", "down_suh", "down_svh")])
    y, ps = ob.moe_rows(bank, G["moe_x"].astype(np.float32), G["moe_inds"], G["moe_scores"], per_slot=True)
    assert np.array_equal(y, G["moe_y"]) and np.array_equal(ps, G["moe_per_slot"])
    yc = ob.moe_rows(bank, G["moe_x"].astype(np.float32), G["moe_inds"], G["moe_scores"], limit=1.0, threads=1)
    assert np.array_equal(yc, G["moe_y_clamped_gate_in_1"])


@pytest.mark.gpu
def test_cuda_path_against_golden():
    import torch

    import turboexl3_b200 as t3
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    bits = lambda t: t.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    for n in RATES:
        trellis = np.tile(G[f"tile_n{n}_words"], 64).reshape(8, 8, n)
        for cb, name, w in ((t3.MUL1, "mul1", 16), (t3.MCG, "mcg", 16), (t3.MCG, "mcg", 12)):
            got = bits(t3.dequantize(dev(trellis), t3.Decode(cb, w)))[:16, :16]
            assert np.array_equal(got, G[f"tile_n{n}_{name}_w{w}"]), (n, name, w)
    for tag, n, cb, w in (("lin_k3_mul1", 48, t3.MUL1, 16), ("lin_n40_mcg_w12", 40, t3.MCG, 12)):
        t, a, b, x = (G[f"{tag}_{k}"] for k in ("trellis", "suh", "svh", "x"))
        dec = t3.Decode(cb, w)
        assert np.array_equal(bits(t3.dequantize(dev(t), dec)), G[f"{tag}_what"])
        y = t3.linear(dev(x), dev(t), dev(a), dev(b), dec).float().cpu().numpy()
        assert ob.compare(y, G[f"{tag}_y"])["max_ratio"] <= 5e-3
        assert ob.compare(y, G[f"{tag}_y"], 2.0 ** -11)["max_ratio"] <= 3e-3
    d = {k: dev(G[f"moe_{k}"]) for k in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh", "up_svh", "down_t",
                                           "down_suh", "down_svh")}
    for k in list(d):
        if k.endswith("_t"):
            d[k] = d[k].view(6, *G[f"moe_{k}"].shape[1:])
    bank = t3.Bank(t3.Proj(d["gate_t"], d["gate_suh"], d["gate_svh"]), t3.Proj(d["up_t"], d["up_suh"], d["up_svh"]),
                   t3.Proj(d["down_t"], d["down_suh"], d["down_svh"]))
    x = dev(G["moe_x"]).view(1, 2, 256)
    inds, scores = dev(G["moe_inds"]).view(1, 2, 3), dev(G["moe_scores"]).view(1, 2, 3)
    y = t3.moe(x, bank, inds, scores).float().cpu().numpy().reshape(2, 256)
    assert ob.compare(y, G["moe_y"], 2.0 ** -11)["max_ratio"] <= 4e-3
    yc = t3.moe_clamped(x, bank, inds, scores, t3.Decode.mul1, 1).float().cpu().numpy().reshape(2, 256)
    assert ob.compare(yc, G["moe_y_clamped_gate_in_1"], 2.0 ** -11)["max_ratio"] <= 4e-3
