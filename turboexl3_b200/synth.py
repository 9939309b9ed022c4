"""Seeded synthetic EXL3 operands (numpy, host side): what stands in for real packs in tests and benches.

Codes are uniform random halfwords (every 16-bit pattern is a valid codeword, as the reference's synthetic banks assume,
src/core/ref.zig:42-44); suh/svh are random signs; activations are N(0, 1). Single linears use magnitude-1 signs; routed
banks scale svh by a power of two near 1/sqrt(in) so the SwiGLU product stays inside f16 (the reference scales by
1/sqrt(in) for the same reason, src/core/ref.zig:66-73)."""
from __future__ import annotations

import numpy as np


def signs(rng: np.random.Generator, shape, magnitude: float = 1.0) -> np.ndarray:
    return (np.where(rng.random(shape) < 0.5, -1.0, 1.0) * magnitude).astype(np.float16)


def pow2_inv_sqrt(in_dim: int) -> float:
    return float(2.0 ** (-round(np.log2(np.sqrt(in_dim)))))


def linear(seed: int, in_dim: int, out_dim: int, n: int, scaled: bool = False):
    """(trellis u16 [in/16, out/16, n], suh f16 [in], svh f16 [out])."""
    rng = np.random.default_rng(seed)
    trellis = rng.integers(0, 65536, (in_dim // 16, out_dim // 16, n), dtype=np.uint16)
    mag = pow2_inv_sqrt(in_dim) if scaled else 1.0
    return trellis, signs(rng, in_dim), signs(rng, out_dim, mag)


def bank(seed: int, experts: int, hidden: int, inter: int, n: int) -> dict:
    """A routed bank's nine arrays, expert-major."""
    rng = np.random.default_rng(seed)
    code = lambda i, o: rng.integers(0, 65536, (experts, i // 16, o // 16, n), dtype=np.uint16)
    return {
        "gate_t": code(hidden, inter), "gate_suh": signs(rng, (experts, hidden)),
        "gate_svh": signs(rng, (experts, inter), pow2_inv_sqrt(hidden)),
        "up_t": code(hidden, inter), "up_suh": signs(rng, (experts, hidden)),
        "up_svh": signs(rng, (experts, inter), pow2_inv_sqrt(hidden)),
        "down_t": code(inter, hidden), "down_suh": signs(rng, (experts, inter)),
        "down_svh": signs(rng, (experts, hidden), pow2_inv_sqrt(inter)),
    }


def routing(seed: int, rows: int, experts: int, topk: int, kind: str = "softmax"):
    """Router logits N(0, 1) -> top-k ids (int32) and renormalised scores (f32): softmax (config 3/4) or sigmoid."""
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((rows, experts)).astype(np.float32)
    probs = np.exp(logits - logits.max(1, keepdims=True)) if kind == "softmax" else 1.0 / (1.0 + np.exp(-logits))
    if kind == "softmax":
        probs = probs / probs.sum(1, keepdims=True)
    inds = np.argsort(-probs, axis=1, kind="stable")[:, :topk].astype(np.int32)
    sc = np.take_along_axis(probs, inds, axis=1)
    sc = (sc / sc.sum(1, keepdims=True)).astype(np.float32)
    return inds, sc


def activations(seed: int, rows: int, dim: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((rows, dim)).astype(np.float16)
