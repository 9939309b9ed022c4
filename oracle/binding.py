"""ctypes binding of the CPU oracle (oracle/t3_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the bench's CPU-baseline legs, never by the
turboexl3_b200 package. Each wrapper names the oracle function it calls; those cite the reference lines they follow.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libt3_oracle.so")

MUL1, MCG = 0, 1
CLAMP_GATE_IN, CLAMP_SILU_OUT = 0, 1


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only)."""
    src = os.path.join(_HERE, "t3_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < max(
        os.path.getmtime(src), os.path.getmtime(os.path.join(_HERE, "t3_oracle.h")))
    if force or stale:
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True, capture_output=True)
    return _LIB_PATH


_lib = None

_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)


class _Bank(C.Structure):
    _fields_ = [("experts", C.c_size_t), ("hidden", C.c_size_t), ("inter", C.c_size_t), ("n", C.c_uint32),
                ("gate_t", _u16p), ("gate_suh", _u16p), ("gate_svh", _u16p),
                ("up_t", _u16p), ("up_suh", _u16p), ("up_svh", _u16p),
                ("down_t", _u16p), ("down_suh", _u16p), ("down_svh", _u16p)]


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        build()
    L = C.CDLL(_LIB_PATH)
    sz, u32, i32, u64, f32, f64 = C.c_size_t, C.c_uint32, C.c_int, C.c_uint64, C.c_float, C.c_double
    sig = {
        "t3o_had_scale": (f32, []),
        "t3o_multiplier": (u32, [i32]),
        "t3o_window_mask": (i32, [i32]),
        "t3o_rate_admitted": (i32, [u64]),
        "t3o_bit_end": (u64, [u32, u64]),
        "t3o_fresh_bits": (u64, [u32, u64]),
        "t3o_f32_to_f16_bits": (C.c_uint16, [f32]),
        "t3o_f16_bits_to_f32": (f32, [C.c_uint16]),
        "t3o_decode_mcg": (C.c_uint16, [C.c_uint16]),
        "t3o_decode_mul1": (C.c_uint16, [C.c_uint16]),
        "t3o_mul1_t": (u32, [C.c_uint16]),
        "t3o_decode_codeword": (C.c_uint16, [C.c_uint16, i32]),
        "t3o_unpack_tile": (None, [_u16p, u32, _u16p]),
        "t3o_stream_bit": (i32, [_u16p, u32, u64]),
        "t3o_codeword_by_definition": (C.c_uint16, [_u16p, u32, u64]),
        "t3o_tensor_core_perm": (None, [_u32p]),
        "t3o_decode_tile": (None, [_u16p, u32, i32, i32, _u16p]),
        "t3o_hadamard128": (None, [_f32p]),
        "t3o_pack_symbols": (None, [_u16p, u32, _u16p]),
        "t3o_reconstruct_inner": (None, [_u16p, sz, sz, u32, i32, i32, _u16p]),
        "t3o_reconstruct_public": (i32, [_u16p, _u16p, _u16p, sz, sz, u32, i32, i32, _u16p]),
        "t3o_prepare_input": (None, [_f32p, _u16p, _f32p, sz]),
        "t3o_inner_gemv": (None, [_u16p, _f32p, sz, sz, u32, i32, i32, _f32p]),
        "t3o_finish_output": (None, [_f32p, _u16p, _f32p, sz]),
        "t3o_project": (None, [_f32p, _u16p, _u16p, _u16p, sz, sz, u32, i32, i32, _f32p, _f32p, _f32p]),
        "t3o_project_what": (None, [_f32p, _u16p, _u16p, _u16p, sz, sz, _f32p, _f32p, _f32p]),
        "t3o_swiglu_clamped": (f32, [f32, f32, f32]),
        "t3o_swiglu_clamped_out": (f32, [f32, f32, f32]),
        "t3o_moe_row": (i32, [C.POINTER(_Bank), i32, i32, f32, i32, _f32p, _u32p, _f32p, sz, _f32p, _f32p]),
        "t3o_compare": (None, [_f32p, _f32p, sz, f64, C.POINTER(f64)]),
        "t3o_linear_rows": (i32, [_f32p, sz, _u16p, _u16p, _u16p, sz, sz, u32, i32, i32, _f32p, i32]),
        "t3o_linear_rows_what": (i32, [_f32p, sz, _u16p, _u16p, _u16p, sz, sz, _f32p, i32]),
        "t3o_moe_rows": (i32, [C.POINTER(_Bank), i32, i32, f32, i32, _f32p, sz, _u32p, _f32p, sz, _f32p, i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _u16(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def host_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


# ---- format.zig scalars -------------------------------------------------------------------------------------------

def decode_table(codebook: int, window_bits: int = 16) -> np.ndarray:
    """All 65,536 codewords decoded (t3o_decode_codeword after the window mask), as f16 bits."""
    L = lib()
    mask = L.t3o_window_mask(window_bits)
    return np.array([L.t3o_decode_codeword(cw & mask, codebook) for cw in range(65536)], dtype=np.uint16)


def unpack_tile(words, n: int) -> np.ndarray:
    w = _u16(words)
    assert w.size == n
    out = np.empty(256, np.uint16)
    lib().t3o_unpack_tile(_p(w, _u16p), n, _p(out, _u16p))
    return out


def codewords_by_definition(words, n: int) -> np.ndarray:
    w = _u16(words)
    L = lib()
    return np.array([L.t3o_codeword_by_definition(_p(w, _u16p), n, t) for t in range(256)], dtype=np.uint16)


def tensor_core_perm() -> np.ndarray:
    out = np.empty(256, np.uint32)
    lib().t3o_tensor_core_perm(_p(out, _u32p))
    return out


def pack_symbols(symbols, k: int) -> np.ndarray:
    s = _u16(symbols)
    out = np.empty(16 * k, np.uint16)
    lib().t3o_pack_symbols(_p(s, _u16p), k, _p(out, _u16p))
    return out


def hadamard128(v) -> np.ndarray:
    a = _f32(v).copy()
    assert a.size == 128
    lib().t3o_hadamard128(_p(a, _f32p))
    return a


# ---- weights and rows ---------------------------------------------------------------------------------------------

def reconstruct_inner(trellis, in_f: int, out_f: int, n: int, codebook: int, window_bits: int = 16) -> np.ndarray:
    """W_hat [in, out] as f16 bits (t3o_reconstruct_inner)."""
    t = _u16(trellis)
    assert t.size == (in_f // 16) * (out_f // 16) * n
    out = np.empty((in_f, out_f), np.uint16)
    lib().t3o_reconstruct_inner(_p(t, _u16p), in_f, out_f, n, codebook, window_bits, _p(out, _u16p))
    return out


def reconstruct_public(trellis, suh, svh, in_f, out_f, n, codebook, window_bits=16) -> np.ndarray:
    t, a, b = _u16(trellis), _u16(suh), _u16(svh)
    out = np.empty((in_f, out_f), np.uint16)
    rc = lib().t3o_reconstruct_public(_p(t, _u16p), _p(a, _u16p), _p(b, _u16p), in_f, out_f, n, codebook,
                                      window_bits, _p(out, _u16p))
    assert rc == 0
    return out


def project(x, trellis, suh, svh, in_f, out_f, n, codebook, window_bits=16, stages: bool = False):
    """One row through t3o_project; with stages=True also the prepared input and the f16-rounded inner product."""
    xv, t, a, b = _f32(x), _u16(trellis), _u16(suh), _u16(svh)
    assert xv.size == in_f and a.size == in_f and b.size == out_f
    tr, inner, y = np.empty(in_f, np.float32), np.empty(out_f, np.float32), np.empty(out_f, np.float32)
    lib().t3o_project(_p(xv, _f32p), _p(t, _u16p), _p(a, _u16p), _p(b, _u16p), in_f, out_f, n, codebook,
                      window_bits, _p(tr, _f32p), _p(inner, _f32p), _p(y, _f32p))
    return (y, tr, inner) if stages else y


def linear_rows(x, trellis, suh, svh, in_f, out_f, n, codebook, window_bits=16, threads: int = 1) -> np.ndarray:
    """Rows of format.project, faithful to the reference: every tile decoded on every row (t3o_linear_rows)."""
    xv, t, a, b = _f32(x).reshape(-1, in_f), _u16(trellis), _u16(suh), _u16(svh)
    y = np.empty((xv.shape[0], out_f), np.float32)
    rc = lib().t3o_linear_rows(_p(xv, _f32p), xv.shape[0], _p(t, _u16p), _p(a, _u16p), _p(b, _u16p), in_f, out_f,
                               n, codebook, window_bits, _p(y, _f32p), threads)
    assert rc == 0
    return y


def linear_rows_what(x, what, suh, svh, in_f, out_f, threads: int = 0) -> np.ndarray:
    """Rows of format.project's values from a W_hat decoded once (t3o_linear_rows_what, ref.zig Linear.row)."""
    xv, w, a, b = _f32(x).reshape(-1, in_f), _u16(what), _u16(suh), _u16(svh)
    assert w.size == in_f * out_f
    y = np.empty((xv.shape[0], out_f), np.float32)
    rc = lib().t3o_linear_rows_what(_p(xv, _f32p), xv.shape[0], _p(w, _u16p), _p(a, _u16p), _p(b, _u16p), in_f,
                                    out_f, _p(y, _f32p), threads or host_threads())
    assert rc == 0
    return y


@dataclass
class Bank:
    """A routed bank as the reference stacks it (ref.zig:9-40): expert e on axis 0 of every array, f16 as bits."""
    experts: int
    hidden: int
    inter: int
    n: int
    gate_t: np.ndarray
    gate_suh: np.ndarray
    gate_svh: np.ndarray
    up_t: np.ndarray
    up_suh: np.ndarray
    up_svh: np.ndarray
    down_t: np.ndarray
    down_suh: np.ndarray
    down_svh: np.ndarray

    def _c(self):
        keep = [_u16(getattr(self, f)) for f in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh", "up_svh",
                                                  "down_t", "down_suh", "down_svh")]
        s = _Bank(self.experts, self.hidden, self.inter, self.n, *[_p(k, _u16p) for k in keep])
        return s, keep


def moe_rows(bank: Bank, x, slots, scores, codebook=MUL1, window_bits=16, limit: float = 0.0,
             clamp_at: int = CLAMP_GATE_IN, threads: int = 0, per_slot: bool = False):
    """Rows of ref.moeRowClampedAt (t3o_moe_rows); y [rows, hidden] f32. per_slot=True (one thread) also returns
    every slot's down projection output [rows, topk, hidden]."""
    xv = _f32(x).reshape(-1, bank.hidden)
    rows = xv.shape[0]
    sl = np.ascontiguousarray(slots, dtype=np.uint32).reshape(rows, -1)
    sc = _f32(scores).reshape(rows, -1)
    topk = sl.shape[1]
    y = np.empty((rows, bank.hidden), np.float32)
    cb, keep = bank._c()
    L = lib()
    if per_slot:
        ps = np.empty((rows, topk, bank.hidden), np.float32)
        for r in range(rows):
            rc = L.t3o_moe_row(C.byref(cb), codebook, window_bits, limit, clamp_at, _p(xv[r], _f32p),
                               _p(sl[r], _u32p), _p(sc[r], _f32p), topk, _p(y[r], _f32p), _p(ps[r], _f32p))
            assert rc == 0
        return y, ps
    rc = L.t3o_moe_rows(C.byref(cb), codebook, window_bits, limit, clamp_at, _p(xv, _f32p), rows, _p(sl, _u32p),
                        _p(sc, _f32p), topk, _p(y, _f32p), threads or host_threads())
    assert rc == 0
    del keep
    return y


def compare(got, ref, half_ulp: float = 0.0) -> dict:
    """ref.compare / ref.compareRounded (t3o_compare)."""
    g, r = _f32(got).ravel(), _f32(ref).ravel()
    assert g.size == r.size
    out = (C.c_double * 3)()
    lib().t3o_compare(_p(g, _f32p), _p(r, _f32p), g.size, half_ulp, out)
    return {"max_abs": out[0], "rms_ref": out[1], "max_ratio": out[2]}
