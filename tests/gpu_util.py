"""Helpers of the GPU parity tests: numpy <-> device, the oracle calls, and the error measures the reference uses
(ref.compare / ref.compareRounded, src/core/ref.zig:195-218)."""
import numpy as np
import torch

from oracle import binding as ob

HALF_ULP_F16 = 2.0 ** -11
HALF_ULP_BF16 = 2.0 ** -8

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def round_to(a: np.ndarray, dt: str) -> np.ndarray:
    """f32 values rounded once to the activation dtype, back in f32 (what a kernel's final store does)."""
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    return t.to(TORCH_DT[dt]).float().numpy()


def x_as(x_f16: np.ndarray, dt: str) -> torch.Tensor:
    """An activation holding the same values in dtype dt (values are f16-representable so every dtype is exact,
    except bf16 which rounds; the oracle is then fed the rounded values)."""
    return torch.from_numpy(x_f16.astype(np.float32)).to(TORCH_DT[dt]).cuda()


def report(got: np.ndarray, ref: np.ndarray, dt: str) -> dict:
    """compare, compareRounded at the dtype's half ulp, and the share of outputs equal bit for bit to the oracle's value
    rounded to the output dtype. The engine multiplies the
    exact f16 weights, so it differs from the oracle only through f32 summation order (the Hadamard butterflies and the
    tensor-core accumulation): a few percent of the f16 roundings inside a projection land on the other side, and each
    moves the outputs of its 128-block by a fraction of an ulp."""
    # an f32 activation still carries an f16-rounded y (the projection rounds y to f16 before the output dtype,
    # docs/core/format.md:27-31), so its rounding allowance is f16's
    half = HALF_ULP_BF16 if dt == "bf16" else HALF_ULP_F16
    ref_r = round_to(ref, dt) if dt != "f32" else ref
    return {
        "compare": ob.compare(got, ref)["max_ratio"],
        "rounded": ob.compare(got, ref, half)["max_ratio"],
        "equal": float(np.mean(got.astype(np.float32) == ref_r.astype(np.float32))),
    }


# Bars. COMPARE is the reference's own (src/core/gpu_test.zig:46,438,446). ROUNDED is this engine's tighter bar on
# compareRounded: a single f16 rounding flip on a 5-sigma output is 2.4e-3 of the RMS after the half ulp is taken off.
COMPARE_BAR = {"f32": 5e-3, "f16": 5e-3, "bf16": 2.5e-2}
ROUNDED_BAR = 3e-3


ACHIEVED = []  # every checked case's measures, in order; written out at the end of the run when T3_PARITY_REPORT names a file


def record(what, r: dict) -> None:
    ACHIEVED.append({"what": repr(what), **{k: float(v) for k, v in r.items()}})


def check(got: np.ndarray, ref: np.ndarray, dt: str, what=None) -> dict:
    r = report(got, ref, dt)
    record(what, r)
    assert np.all(np.isfinite(got)), what
    assert r["compare"] <= COMPARE_BAR[dt], (what, r)
    assert r["rounded"] <= ROUNDED_BAR, (what, r)
    if dt == "f16":
        assert r["equal"] >= 0.5, (what, r)  # most outputs are the oracle's bits; the rest are one rounding away
    return r
