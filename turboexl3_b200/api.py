"""Host-side mirror of turboexl3's module API (src/root.zig) over the C ABI in include/t3.h.

Same names and argument meaning as the reference: `linear(x, trellis, suh, svh, dec)` (src/root.zig:309),
`moe(x, bank, inds, scores, dec)` (:822), `moe_swiglu` (:831), `moe_clamped` (:1001), `moe_with_shared` (:976),
`configure` (src/core/config.zig:175), and the refusals under the reference's error names. Torch is only the holder of
device memory and streams here; every computation is a kernel of libt3.so, and a missing library is an error, never a
fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional
from dataclasses import dataclass

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libt3.so")

MUL1, MCG = 0, 1
CLAMP_GATE_IN, CLAMP_SILU_OUT = 0, 1
DECODE_ROWS_MAX = 32
REDUCE_MAX_TOPK = 32

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class Exl3Error(RuntimeError):
    """A refusal or failure of the engine; `.name` is the reference's error name (e.g. "BadExl3Shape")."""

    def __init__(self, status: int, name: str):
        super().__init__(f"{name} (status {status})")
        self.status = status
        self.name = name


class _Decode(C.Structure):
    _fields_ = [("codebook", C.c_int), ("window_bits", C.c_int)]


class _Proj(C.Structure):
    _fields_ = [("trellis", C.c_void_p), ("suh", C.c_void_p), ("svh", C.c_void_p)]


class _Bank(C.Structure):
    _fields_ = [("gate", _Proj), ("up", _Proj), ("down", _Proj), ("experts", C.c_int), ("hidden", C.c_int),
                ("inter", C.c_int), ("n_gate", C.c_int), ("n_up", C.c_int), ("n_down", C.c_int)]


class _Spec(C.Structure):
    _fields_ = [("n", C.c_uint32), ("codebook", C.c_int), ("window_bits", C.c_int)]


class Launch(C.Structure):
    """t3_launch: one kernel launch of a plan (symbol, group, grid, block, shared bytes, cluster size, buffer roles)."""
    _fields_ = [("symbol", C.c_char * 64), ("group", C.c_char * 16), ("grid", C.c_uint32 * 3), ("block", C.c_uint32),
                ("shared", C.c_uint32), ("cluster", C.c_uint32), ("nroles", C.c_int), ("roles", C.c_int * 24)]


class _Config(C.Structure):
    _fields_ = [("prefill", C.c_int), ("ring_bytes", C.c_uint32), ("dense_split", C.c_uint32), ("no_overlap", C.c_int),
                ("probe", C.c_int)]


# every symbol include/t3.h declares: (restype, argtypes)
_vp, _sz, _i, _u32 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32
SYMBOLS = {
    "t3_status_name": (C.c_char_p, [_i]),
    "t3_uses_prefill_arm": (_i, [_sz]),
    "t3_admit_topk": (_i, [_u32]),
    "t3_trellis_admitted": (_i, [C.POINTER(C.c_int), _i, _u32, _u32, _u32, _u32]),
    "t3_parse_expert_quant": (_i, [C.c_char_p, _sz, C.POINTER(_Spec)]),
    "t3_config_default": (None, [C.POINTER(_Config)]),
    "t3_configure": (_i, [C.POINTER(_Config)]),
    "t3_device_error": (_i, [_vp, C.POINTER(_u32), _i]),
    "t3_selftest_wait_runs_out": (_i, [_vp]),
    "t3_dequant": (_i, [_vp, _i, _i, _i, _Decode, _vp, _vp]),
    "t3_codebook_table": (_i, [_Decode, _vp, _vp]),
    "t3_linear_workspace_bytes": (_sz, [_sz, _i, _i, _i]),
    "t3_linear": (_i, [_vp, _i, _sz, _vp, _vp, _vp, _i, _i, _i, _Decode, _vp, _vp, _sz, _vp]),
    "t3_moe_workspace_bytes": (_sz, [_sz, _i, C.POINTER(_Bank)]),
    "t3_moe": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _vp, _i, _i, _Decode, _vp, _vp, _sz, _vp]),
    "t3_moe_swiglu": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _vp, _i, _i, _Decode, _u32, _i, _vp, _vp, _sz, _vp]),
    "t3_moe_clamped": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _vp, _i, _i, _Decode, _i, _vp, _vp, _sz, _vp]),
    "t3_moe_with_shared": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _vp, _i, _i, _Decode, _vp, _vp, _vp, _sz, _vp]),
    "t3_moe_swiglu_rows": (_i, [_vp, _i, _sz, _vp, _sz, C.POINTER(_Bank), _vp, _vp, _i, _Decode, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "t3_moe_with_shared_after": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _vp, _i, _i, _Decode, _vp, _vp, _vp, _vp, _sz, _vp]),
    "t3_moe_merge": (_i, [_vp, _vp, _i, _sz, _i, _i, _vp, _vp, _i, _vp]),
    "t3_moe_merge_mapped": (_i, [_vp, _vp, _vp, _i, _sz, _i, _i, _vp, _vp, _i, _vp]),
    "t3_ep_plan": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "t3_moe_noalloc": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _vp, _i, _i, _Decode, _vp, _vp]),
    "t3_set_trace": (None, [_vp]),
    "t3_launch_count": (C.c_uint64, []),
    "t3_resident_bytes": (_sz, [_i, _i]),
    "t3_resident_build": (_i, [_vp, _i, _i, _i, _Decode, _vp, _vp]),
    "t3_linear_resident": (_i, [_vp, _i, _sz, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "t3_unrot_build": (_i, [_vp, _vp, _vp, _i, _i, _i, _Decode, _i, _vp, _vp]),
    "t3_linear_unrot": (_i, [_vp, _i, _sz, _vp, _i, _i, _vp, _vp]),
    "t3_moe_clamped_banked": (_i, [_vp, _i, _sz, C.POINTER(_Bank), _vp, _Decode, _i, _vp, _i, _vp, _sz, _vp]),
    "t3_plan_linear": (_i, [_sz, _i, _i, _i, _Decode, C.POINTER(Launch), _i]),
    "t3_plan_moe": (_i, [_sz, _i, C.POINTER(_Bank), _Decode, C.POINTER(Launch), _i]),
    "t3_last_kernel_symbol": (C.c_char_p, []),
    "t3_engines_held": (None, [_vp]),
    "t3_release_engines": (None, []),
}

_lib = None


def lib() -> C.CDLL:
    """libt3.so, loaded once. Raises when it has not been built: there is no other implementation to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} is missing: build it with `python -m turboexl3_b200.build` "
                               "(this package has no CPU or PyTorch fallback)")
        L = C.CDLL(_LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def status_name(status: int) -> str:
    return lib().t3_status_name(status).decode()


def _check(status: int) -> None:
    if status != 0:
        raise Exl3Error(status, status_name(status))


@dataclass(frozen=True)
class Decode:
    """format.Decode (src/core/format.zig:72-78)."""
    codebook: int = MUL1
    window_bits: int = 16

    def _c(self) -> _Decode:
        return _Decode(self.codebook, self.window_bits)


Decode.mul1 = Decode(MUL1)
Decode.mcg = Decode(MCG)


@dataclass
class Proj:
    """root.Proj (src/root.zig:74): trellis U16/I16 [E, in/16, out/16, n], suh F16 [E, in], svh F16 [E, out]."""
    trellis: torch.Tensor
    suh: torch.Tensor
    svh: torch.Tensor


@dataclass
class Bank:
    """root.Bank (src/root.zig:75)."""
    gate: Proj
    up: Proj
    down: Proj


def _stream_ptr(x: torch.Tensor) -> int:
    return torch.cuda.current_stream(x.device).cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("turboexl3_b200 takes CUDA tensors only")
        if not t.is_contiguous():
            raise RuntimeError("turboexl3_b200 takes contiguous tensors")


def _trellis_ok(t: torch.Tensor) -> bool:
    return t.dtype in (torch.uint16, torch.int16)


def configure(prefill: bool = True, ring_bytes: int = 0, dense_split: int = 0, no_overlap: bool = False, probe: int = 0) -> None:
    """core.config.configure (src/core/config.zig:175): process-wide, before the first call. probe 1..3 swaps the dense
    decode-row kernel for a timing probe (see t3_config in include/t3.h): measurements only."""
    cfg = _Config(int(prefill), ring_bytes, dense_split, int(no_overlap), int(probe))
    _check(lib().t3_configure(C.byref(cfg)))


def device_error(clear: bool = True) -> int:
    """Bits set by kernels whose bounded waits ran out (0 = none). Synchronises the current stream."""
    bits = C.c_uint32(0)
    _check(lib().t3_device_error(torch.cuda.current_stream().cuda_stream, C.byref(bits), int(clear)))
    return bits.value


def plan_linear(rows: int, in_dim: int, out_dim: int, n: int, dec: "Decode" = None) -> list:
    """t3_plan_linear: the launches a decode-row `linear` records, as dicts (symbol, group, grid, block, shared, cluster, roles)."""
    out = (Launch * 4)()
    k = lib().t3_plan_linear(rows, in_dim, out_dim, n, (dec or Decode.mul1)._c(), out, 4)
    if k < 0:
        _check(-k)
    return [_launch_dict(out[i]) for i in range(k)]


def plan_moe(rows: int, topk: int, experts: int, hidden: int, inter: int, n: int, dec: "Decode" = None) -> list:
    """t3_plan_moe for a bank geometry (no device memory needed)."""
    bank = _Bank(_Proj(), _Proj(), _Proj(), experts, hidden, inter, n, n, n)
    out = (Launch * 4)()
    k = lib().t3_plan_moe(rows, topk, C.byref(bank), (dec or Decode.mul1)._c(), out, 4)
    if k < 0:
        _check(-k)
    return [_launch_dict(out[i]) for i in range(k)]


def _launch_dict(l: Launch) -> dict:
    return {"symbol": l.symbol.decode(), "group": l.group.decode(), "grid": tuple(l.grid), "block": l.block, "shared": l.shared,
            "cluster": l.cluster, "roles": [l.roles[i] for i in range(l.nroles)]}


def last_kernel_symbol() -> str:
    return lib().t3_last_kernel_symbol().decode()


def launch_count() -> int:
    return int(lib().t3_launch_count())


def engines_held() -> dict:
    """root.enginesHeld (src/root.zig:1183-1192): distinct geometries served per path since the last release."""
    out = (C.c_size_t * 3)()
    lib().t3_engines_held(out)
    return {"decode": int(out[0]), "dense": int(out[1]), "prefill": int(out[2])}


def release_engines() -> None:
    """root.releaseEngines (src/root.zig:1148-1181)."""
    lib().t3_release_engines()


def parse_expert_quant(json_text: str) -> dict:
    """spec.parseExpertQuant (src/core/spec.zig:38-50)."""
    raw = json_text.encode()
    spec = _Spec()
    _check(lib().t3_parse_expert_quant(raw, len(raw), C.byref(spec)))
    return {"n": spec.n, "codebook": spec.codebook, "window_bits": spec.window_bits}


def trellis_admitted(shape, experts: int, in_dim: int, out_dim: int, n: int) -> bool:
    arr = (C.c_int * len(shape))(*shape)
    return bool(lib().t3_trellis_admitted(arr, len(shape), experts, in_dim, out_dim, n))


def codebook_table(dec: Decode, device="cuda") -> torch.Tensor:
    """All 65,536 codewords through the device decoders (f16 bits as int16 storage viewed uint16 on the host)."""
    out = torch.empty(65536, dtype=torch.int16, device=device)
    _check(lib().t3_codebook_table(dec._c(), out.data_ptr(), _stream_ptr(out)))
    return out


def dequantize(trellis: torch.Tensor, dec: Decode = Decode.mul1) -> torch.Tensor:
    """W_hat f16 [in, out] (Dense.dequantize, src/core/dense.zig:909-922)."""
    _need_cuda(trellis)
    if trellis.dim() != 3:
        raise Exl3Error(1, "BadExl3Shape")
    if not _trellis_ok(trellis):
        raise Exl3Error(2, "BadExl3Dtype")
    in_dim, out_dim, n = trellis.shape[0] * 16, trellis.shape[1] * 16, trellis.shape[2]
    w = torch.empty((in_dim, out_dim), dtype=torch.float16, device=trellis.device)
    _check(lib().t3_dequant(trellis.data_ptr(), in_dim, out_dim, n, dec._c(), w.data_ptr(), _stream_ptr(trellis)))
    return w


def linear(x: torch.Tensor, trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor,
           dec: Decode = Decode.mul1) -> torch.Tensor:
    """root.linear (src/root.zig:309-351): y [..., out] in x's dtype for x [..., in]."""
    _need_cuda(x, trellis, suh, svh)
    if x.dim() < 1 or trellis.dim() != 3:
        raise Exl3Error(1, "BadExl3Shape")
    in_dim, out_dim, n = trellis.shape[0] * 16, trellis.shape[1] * 16, trellis.shape[2]
    if x.shape[-1] != in_dim or suh.numel() != in_dim or svh.numel() != out_dim:
        raise Exl3Error(1, "BadExl3Shape")
    if x.dtype not in _DTYPES or not _trellis_ok(trellis) or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise Exl3Error(2, "BadExl3Dtype")
    rows = x.numel() // in_dim
    if rows < 1:
        raise Exl3Error(1, "BadExl3Shape")
    y = torch.empty(x.shape[:-1] + (out_dim,), dtype=x.dtype, device=x.device)
    L = lib()
    ws_bytes = L.t3_linear_workspace_bytes(rows, in_dim, out_dim, n)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
    _check(L.t3_linear(x.data_ptr(), _DTYPES[x.dtype], rows, trellis.data_ptr(), suh.data_ptr(), svh.data_ptr(),
                       in_dim, out_dim, n, dec._c(), y.data_ptr(), ws.data_ptr() if ws is not None else None,
                       ws_bytes, _stream_ptr(x)))
    return y


def resident_build(trellis: torch.Tensor, dec: Decode = Decode.mul1) -> torch.Tensor:
    """The kept weight of a trunk linear (t3_resident_build): W_hat transposed, f16 [out, in], decoded once."""
    _need_cuda(trellis)
    if trellis.dim() != 3:
        raise Exl3Error(1, "BadExl3Shape")
    if not _trellis_ok(trellis):
        raise Exl3Error(2, "BadExl3Dtype")
    in_dim, out_dim, n = trellis.shape[0] * 16, trellis.shape[1] * 16, trellis.shape[2]
    L = lib()
    if L.t3_resident_bytes(in_dim, out_dim) != in_dim * out_dim * 2:
        raise Exl3Error(1, "BadExl3Shape")
    w_t = torch.empty((out_dim, in_dim), dtype=torch.float16, device=trellis.device)
    _check(L.t3_resident_build(trellis.data_ptr(), in_dim, out_dim, n, dec._c(), w_t.data_ptr(), _stream_ptr(trellis)))
    return w_t


def linear_resident(x: torch.Tensor, w_hat_t: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor) -> torch.Tensor:
    """linear on a kept weight (t3_linear_resident), more than 32 rows: the same bytes as `linear` on the trellis."""
    _need_cuda(x, w_hat_t, suh, svh)
    if x.dim() < 1 or w_hat_t.dim() != 2:
        raise Exl3Error(1, "BadExl3Shape")
    out_dim, in_dim = w_hat_t.shape
    if x.shape[-1] != in_dim or suh.numel() != in_dim or svh.numel() != out_dim or not w_hat_t.is_contiguous():
        raise Exl3Error(1, "BadExl3Shape")
    if x.dtype not in _DTYPES or w_hat_t.dtype != torch.float16 or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise Exl3Error(2, "BadExl3Dtype")
    rows = x.numel() // in_dim
    y = torch.empty(x.shape[:-1] + (out_dim,), dtype=x.dtype, device=x.device)
    L = lib()
    ws_bytes = L.t3_linear_workspace_bytes(max(rows, 33), in_dim, out_dim, 16)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    _check(L.t3_linear_resident(x.data_ptr(), _DTYPES[x.dtype], rows, w_hat_t.data_ptr(), suh.data_ptr(), svh.data_ptr(),
                                in_dim, out_dim, y.data_ptr(), ws.data_ptr(), ws_bytes, _stream_ptr(x)))
    return y


def _bank_c(bank: Bank, hidden: int) -> _Bank:
    g, u, d = bank.gate, bank.up, bank.down
    for p in (g, u, d):
        _need_cuda(p.trellis, p.suh, p.svh)
        if p.trellis.dim() != 4:
            raise Exl3Error(1, "BadExl3Shape")
        if not _trellis_ok(p.trellis) or p.suh.dtype != torch.float16 or p.svh.dtype != torch.float16:
            raise Exl3Error(2, "BadExl3Dtype")
    experts, inter = g.trellis.shape[0], g.trellis.shape[2] * 16

    def shape_ok(p: Proj, i: int, o: int) -> bool:  # root.validateProjectionAs, src/root.zig:93-101
        return (tuple(p.trellis.shape[:3]) == (experts, i // 16, o // 16) and tuple(p.suh.shape) == (experts, i)
                and tuple(p.svh.shape) == (experts, o))

    if hidden % 128 or inter % 128 or not (shape_ok(g, hidden, inter) and shape_ok(u, hidden, inter)
                                           and shape_ok(d, inter, hidden)):
        raise Exl3Error(1, "BadExl3Shape")
    mk = lambda p: _Proj(p.trellis.data_ptr(), p.suh.data_ptr(), p.svh.data_ptr())
    return _Bank(mk(g), mk(u), mk(d), experts, hidden, inter, g.trellis.shape[3], u.trellis.shape[3],
                 d.trellis.shape[3])


def _moe(x, bank, inds, scores, dec, limit, clamp_at, shared, entry: str, shared_ready=None):
    _need_cuda(x, inds, scores)
    if x.dim() != 3 or inds.dim() != 3 or x.shape[:2] != inds.shape[:2] or inds.shape != scores.shape:
        raise Exl3Error(1, "BadExl3Shape")  # root.validateCall, src/root.zig:128-141
    topk = inds.shape[2]
    if topk <= 0 or topk > REDUCE_MAX_TOPK or x.shape[2] % 128:
        raise Exl3Error(1, "BadExl3Shape")
    if x.dtype not in _DTYPES or inds.dtype not in (torch.int32, torch.uint32) or scores.dtype not in _DTYPES:
        raise Exl3Error(2, "BadExl3Dtype")
    hidden = x.shape[2]
    cb = _bank_c(bank, hidden)
    rows = x.shape[0] * x.shape[1]
    if shared is not None:
        _need_cuda(shared)
        if shared.dtype != x.dtype or shared.numel() != x.numel():
            raise Exl3Error(1, "BadExl3Shape")
    L = lib()
    ws_bytes = L.t3_moe_workspace_bytes(rows, topk, C.byref(cb))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    y = torch.empty_like(x)
    common = (x.data_ptr(), _DTYPES[x.dtype], rows, C.byref(cb), inds.data_ptr(), scores.data_ptr(),
              _DTYPES[scores.dtype], topk, dec._c())
    tail = (y.data_ptr(), ws.data_ptr(), ws_bytes, _stream_ptr(x))
    if entry == "moe":
        _check(L.t3_moe(*common, *tail))
    elif entry == "swiglu":
        _check(L.t3_moe_swiglu(*common, limit, clamp_at, *tail))
    elif entry == "clamped":
        _check(L.t3_moe_clamped(*common, limit, *tail))
    elif shared_ready is not None:
        _check(L.t3_moe_with_shared_after(*common, shared.data_ptr(), shared_ready.cuda_event, *tail))
    else:
        _check(L.t3_moe_with_shared(*common, shared.data_ptr(), *tail))
    return y


def moe(x, bank: Bank, inds, scores, dec: Decode = Decode.mul1, verify_rows: bool = False) -> torch.Tensor:
    """root.moe (src/root.zig:822-825): x [B, S, D], inds/scores [B, S, K]; y in x's shape and dtype."""
    del verify_rows  # accepted and ignored, as the reference does
    return _moe(x, bank, inds, scores, dec, 0, CLAMP_GATE_IN, None, "moe")


def moe_swiglu_rows(x: torch.Tensor, rows: torch.Tensor, bank: Bank, inds: torch.Tensor, scores: torch.Tensor,
                    dec: Decode = Decode.mul1, limit: int = 0, clamp_at: int = CLAMP_GATE_IN,
                    out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """root.moeSwigluRows (src/root.zig:1007-1021; moeClampedRows at limit 1..128): x [n, hidden], rows u32/i32 [S], inds
    [S], scores [S]; y [S, hidden] in out_dtype (default x's)."""
    _need_cuda(x, rows, inds, scores)
    if x.dim() != 2 or rows.dim() != 1 or rows.shape != inds.shape or rows.shape != scores.shape or x.shape[1] % 128:
        raise Exl3Error(1, "BadExl3Shape")
    out_dtype = out_dtype or x.dtype
    if (x.dtype not in _DTYPES or out_dtype not in _DTYPES or rows.dtype not in (torch.int32, torch.uint32)
            or inds.dtype not in (torch.int32, torch.uint32) or scores.dtype not in _DTYPES):
        raise Exl3Error(2, "BadExl3Dtype")
    cb = _bank_c(bank, x.shape[1])
    S = rows.shape[0]
    L = lib()
    ws_bytes = L.t3_moe_workspace_bytes(S, 1, C.byref(cb))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    y = torch.empty((S, x.shape[1]), dtype=out_dtype, device=x.device)
    _check(L.t3_moe_swiglu_rows(x.data_ptr(), _DTYPES[x.dtype], x.shape[0], rows.data_ptr(), S, C.byref(cb), inds.data_ptr(),
                                scores.data_ptr(), _DTYPES[scores.dtype], dec._c(), limit, clamp_at, y.data_ptr(),
                                _DTYPES[out_dtype], ws.data_ptr(), ws_bytes, _stream_ptr(x)))
    return y


BANKED_ROWS_MAX = 64
BANKED_SKIP_ID = 0xFFFFFFFF


def moe_clamped_banked(x: torch.Tensor, banks, ids: torch.Tensor, dec: Decode = Decode.mul1, limit: int = 7,
                       out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """deepseek_v41.moeClampedBanked / moeClampedBankedAs (src/models/deepseek_v41/api.zig:173-218): x [rows, hidden], banks
    three `Bank`s of one geometry, ids u32/i32 [rows] packed (bank << 24 | slot); y [rows, hidden] in out_dtype (f32 as
    the reference's plain entry), each row its pair's output at weight 1; an id of BANKED_SKIP_ID gives a zero row."""
    _need_cuda(x, ids)
    if x.dim() != 2 or ids.dim() != 1 or ids.shape[0] != x.shape[0] or len(banks) != 3 or x.shape[1] % 128:
        raise Exl3Error(1, "BadExl3Shape")
    if x.dtype not in _DTYPES or out_dtype not in _DTYPES or ids.dtype not in (torch.int32, torch.uint32):
        raise Exl3Error(2, "BadExl3Dtype")
    cbs = (_Bank * 3)(*[_bank_c(b, x.shape[1]) for b in banks])
    rows = x.shape[0]
    L = lib()
    ws_bytes = L.t3_moe_workspace_bytes(min(max(rows, 1), 32), 1, C.byref(cbs[0]))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    y = torch.empty((rows, x.shape[1]), dtype=out_dtype, device=x.device)
    _check(L.t3_moe_clamped_banked(x.data_ptr(), _DTYPES[x.dtype], rows, cbs, ids.data_ptr(), dec._c(), limit, y.data_ptr(),
                                   _DTYPES[out_dtype], ws.data_ptr(), ws_bytes, _stream_ptr(x)))
    return y


def unrot_build(trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor, dec: Decode = Decode.mul1,
                dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """A trunk linear out of the Hadamard basis (t3_unrot_build; root.trunkUnrot, src/root.zig:392-420): W_std transposed,
    [out, in] in `dtype` (f16 or bf16), W_std = diag(suh) H W_hat H diag(svh)."""
    _need_cuda(trellis, suh, svh)
    if trellis.dim() != 3:
        raise Exl3Error(1, "BadExl3Shape")
    in_dim, out_dim, n = trellis.shape[0] * 16, trellis.shape[1] * 16, trellis.shape[2]
    if suh.numel() != in_dim or svh.numel() != out_dim:
        raise Exl3Error(1, "BadExl3Shape")
    if not _trellis_ok(trellis) or suh.dtype != torch.float16 or svh.dtype != torch.float16 or dtype not in (torch.float16, torch.bfloat16):
        raise Exl3Error(2, "BadExl3Dtype")
    w = torch.empty((out_dim, in_dim), dtype=dtype, device=trellis.device)
    _check(lib().t3_unrot_build(trellis.data_ptr(), suh.data_ptr(), svh.data_ptr(), in_dim, out_dim, n, dec._c(), _DTYPES[dtype],
                                w.data_ptr(), _stream_ptr(trellis)))
    return w


def linear_unrot(x: torch.Tensor, w_std_t: torch.Tensor) -> torch.Tensor:
    """y = x W_std on an un-rotated weight (t3_linear_unrot; dense.residentPlain, src/core/dense.zig:1261-1263): more than
    32 rows, x in the weight's dtype, one tensor-core GEMM."""
    _need_cuda(x, w_std_t)
    if x.dim() < 1 or w_std_t.dim() != 2 or x.shape[-1] != w_std_t.shape[1] or not w_std_t.is_contiguous() or not x.is_contiguous():
        raise Exl3Error(1, "BadExl3Shape")
    if x.dtype != w_std_t.dtype or x.dtype not in (torch.float16, torch.bfloat16):
        raise Exl3Error(2, "BadExl3Dtype")
    out_dim, in_dim = w_std_t.shape
    rows = x.numel() // in_dim
    y = torch.empty(x.shape[:-1] + (out_dim,), dtype=x.dtype, device=x.device)
    _check(lib().t3_linear_unrot(x.data_ptr(), _DTYPES[x.dtype], rows, w_std_t.data_ptr(), in_dim, out_dim, y.data_ptr(), _stream_ptr(x)))
    return y


def moe_merge(v: torch.Tensor, scores: torch.Tensor, out_dtype: torch.dtype, shared=None, where=None) -> torch.Tensor:
    """The routed chain's last step (t3_moe_merge / t3_moe_merge_mapped): v f16 [rows, topk, hidden] (with `where`, u32/i32
    [rows * topk]: v [rows * topk, hidden] in any order, slot s's row at v[where[s]]), scores [rows, topk]; y [rows, hidden]."""
    _need_cuda(v, scores)
    rows, topk = scores.shape
    hidden = v.shape[-1]
    if v.dtype != torch.float16 or not v.is_contiguous() or v.numel() != rows * topk * hidden:
        raise Exl3Error(1, "BadExl3Shape")
    if where is not None and (where.numel() != rows * topk or where.dtype not in (torch.int32, torch.uint32)):
        raise Exl3Error(1, "BadExl3Shape")
    y = torch.empty((rows, hidden), dtype=out_dtype, device=v.device)
    _check(lib().t3_moe_merge_mapped(v.data_ptr(), where.data_ptr() if where is not None else None, scores.data_ptr(),
                                     _DTYPES[scores.dtype], rows, topk, hidden,
                                     shared.data_ptr() if shared is not None else None, y.data_ptr(), _DTYPES[out_dtype],
                                     _stream_ptr(v)))
    return y


EP_WORLD_MAX = 8


def ep_plan(inds: torch.Tensor, experts: int, world: int):
    """t3_ep_plan: (order, where, send_rows, meta, counts) for inds [rows, topk] of global expert ids; device tensors, no
    host read."""
    _need_cuda(inds)
    if inds.dim() != 2 or inds.dtype not in (torch.int32, torch.uint32) or not inds.is_contiguous():
        raise Exl3Error(1, "BadExl3Shape")
    rows, topk = inds.shape
    S = rows * topk
    dev = inds.device
    order = torch.empty(S, dtype=torch.int32, device=dev)
    where = torch.empty(S, dtype=torch.int32, device=dev)
    send_rows = torch.empty(S, dtype=torch.int32, device=dev)
    meta = torch.empty((S, 2), dtype=torch.int32, device=dev)
    counts = torch.empty((2, world), dtype=torch.int32, device=dev)
    _check(lib().t3_ep_plan(inds.data_ptr(), rows, topk, experts, world, order.data_ptr(), where.data_ptr(), send_rows.data_ptr(),
                            meta.data_ptr(), counts.data_ptr(), _stream_ptr(inds)))
    return order, where, send_rows, meta, counts


def moe_swiglu(x, bank: Bank, inds, scores, dec: Decode, limit: int, clamp_at: int = CLAMP_GATE_IN) -> torch.Tensor:
    """root.moeSwiglu (src/root.zig:831-833)."""
    return _moe(x, bank, inds, scores, dec, limit, clamp_at, None, "swiglu")


def moe_clamped(x, bank: Bank, inds, scores, dec: Decode, limit: int) -> torch.Tensor:
    """root.moeClamped (src/root.zig:1001-1004): limit in 1..128, else InvalidExl3Clamp."""
    return _moe(x, bank, inds, scores, dec, limit, CLAMP_GATE_IN, None, "clamped")


def moe_with_shared(x, bank: Bank, inds, scores, dec: Decode, shared: torch.Tensor,
                    verify_rows: bool = False, shared_ready: Optional[torch.cuda.Event] = None) -> torch.Tensor:
    """root.moeWithShared (src/root.zig:976-984). shared_ready: an event recorded on the stream that computes `shared`;
    only the call's last launch waits for it (t3_moe_with_shared_after)."""
    del verify_rows
    return _moe(x, bank, inds, scores, dec, 0, CLAMP_GATE_IN, shared, "shared", shared_ready)
