"""ctypes view of the quant-plugin table (include/t3_table.h), the host-buffer face of the engine: what a host
application binds where the reference's host binds `abi.QuantTable` (turboexl3 table/table.zig:30-60). numpy arrays go
in and come out; weights are uploaded once by `load_tensor` / `load_bank`."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import api

VERDICT_OK, VERDICT_UNSUPPORTED, VERDICT_FAILED = 0, 1, 2
CLAIM_NO, CLAIM_BY_MARKER = 0, 1

_NP_DTYPE = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.uint16): 3, np.dtype(np.int16): 4,
             np.dtype(np.int32): 5, np.dtype(np.uint32): 6}
BF16 = 2  # numpy has no bfloat16: pass a uint16 array and dtype=BF16


class Verdict(C.Structure):
    _fields_ = [("kind", C.c_int), ("reason", C.c_char_p)]

    @property
    def ok(self) -> bool:
        return self.kind == VERDICT_OK

    @property
    def why(self) -> str:
        return self.reason.decode() if self.reason else ""


class Array(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("ndim", C.c_int), ("shape", C.c_int64 * 8),
                ("device", C.c_int)]


class Weight(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("layout", C.c_int),
                ("flags", C.c_int), ("block", C.c_int), ("experts", C.c_int), ("in_dim", C.c_int),
                ("out_dim", C.c_int), ("bytes", C.c_size_t)]


class LoadCtx(C.Structure):
    _fields_ = [("block_json", C.c_char_p), ("state", C.c_void_p)]


class SwigluOpts(C.Structure):
    _fields_ = [("limit", C.c_int), ("verify_rows", C.c_int)]


_AP, _WP, _LP = C.POINTER(Array), C.POINTER(Weight), C.POINTER(LoadCtx)


class QuantTable(C.Structure):
    _fields_ = [
        ("name", C.c_char_p),
        ("claims", C.CFUNCTYPE(C.c_int, C.c_char_p, C.c_char_p)),
        ("validate", C.CFUNCTYPE(Verdict, C.c_char_p, C.c_char_p)),
        ("bill", C.CFUNCTYPE(C.c_uint64, C.c_char_p, C.c_char_p, C.c_uint64)),
        ("open", C.CFUNCTYPE(Verdict, _LP)),
        ("close", C.CFUNCTYPE(None, _LP)),
        ("load_tensor", C.CFUNCTYPE(Verdict, _LP, _AP, _AP, _AP, C.c_uint32, _WP)),
        ("load_bank", C.CFUNCTYPE(Verdict, _LP, _AP, _AP, _AP, C.c_uint32, _WP)),
        ("release", C.CFUNCTYPE(None, _WP)),
        ("matmul", C.CFUNCTYPE(Verdict, _WP, _AP, C.c_void_p, _AP)),
        ("moe", C.CFUNCTYPE(Verdict, _WP, _AP, _AP, _AP, C.c_int, C.c_void_p, _AP)),
        ("swiglu", C.CFUNCTYPE(Verdict, _WP, _WP, _WP, _AP, _AP, _AP, C.POINTER(SwigluOpts), C.c_void_p, _AP)),
    ]


TABLE_SYMBOLS = ("t3_table", "t3_table_staging_bytes", "t3_table_release_staging")

_table = None


def table() -> QuantTable:
    global _table
    if _table is None:
        L = api.lib()
        L.t3_table.restype = C.POINTER(QuantTable)
        L.t3_table.argtypes = []
        L.t3_table_staging_bytes.restype = C.c_size_t
        L.t3_table_release_staging.restype = None
        _table = L.t3_table().contents
    return _table


def host_array(a: np.ndarray, dtype: int | None = None) -> Array:
    """An Array over a numpy array's memory (the numpy array must outlive it)."""
    assert a.flags["C_CONTIGUOUS"]
    arr = Array()
    arr.data = a.ctypes.data
    arr.dtype = _NP_DTYPE[a.dtype] if dtype is None else dtype
    arr.ndim = a.ndim
    for i, d in enumerate(a.shape):
        arr.shape[i] = d
    arr.device = 0
    return arr


def device_array(ptr: int, dtype: int, shape) -> Array:
    arr = Array()
    arr.data = ptr
    arr.dtype = dtype
    arr.ndim = len(shape)
    for i, d in enumerate(shape):
        arr.shape[i] = d
    arr.device = 1
    return arr


class Block:
    """An opened block (`open` ... `close`) that loads weights."""

    def __init__(self, block_json: str):
        self._json = block_json.encode()
        self.ctx = LoadCtx(self._json, None)
        self.verdict = table().open(C.byref(self.ctx))

    def close(self) -> None:
        table().close(C.byref(self.ctx))

    def load_tensor(self, trellis: np.ndarray, suh: np.ndarray, svh: np.ndarray, in_dim: int = 0):
        w = Weight()
        v = table().load_tensor(C.byref(self.ctx), C.byref(host_array(trellis)), C.byref(host_array(suh)),
                                C.byref(host_array(svh)), in_dim, C.byref(w))
        return v, w

    def load_bank(self, trellis: np.ndarray, suh: np.ndarray, svh: np.ndarray, in_dim: int = 0):
        w = Weight()
        v = table().load_bank(C.byref(self.ctx), C.byref(host_array(trellis)), C.byref(host_array(suh)),
                              C.byref(host_array(svh)), in_dim, C.byref(w))
        return v, w


def matmul(w: Weight, x: np.ndarray, stream: int = 0, dtype: int | None = None):
    """`matmul` on host arrays: returns (verdict, y) with y a new numpy array of x's dtype."""
    y = np.empty(x.shape[:-1] + (w.out_dim,), x.dtype)
    out = host_array(y, dtype)
    v = table().matmul(C.byref(w), C.byref(host_array(x, dtype)), stream, C.byref(out))
    return v, y


def swiglu(gate: Weight, up: Weight, down: Weight, x: np.ndarray, inds: np.ndarray, scores: np.ndarray,
           limit: int = 0, stream: int = 0):
    y = np.empty_like(x)
    out = host_array(y)
    opts = SwigluOpts(limit, 0)
    v = table().swiglu(C.byref(gate), C.byref(up), C.byref(down), C.byref(host_array(x)), C.byref(host_array(inds)),
                       C.byref(host_array(scores)), C.byref(opts), stream, C.byref(out))
    return v, y
