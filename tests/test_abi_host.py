"""CPU-only checks of the C ABI: libt3.so loads, exports every function include/t3.h declares, and refuses bad calls
before touching the device, under the reference's error names (src/root.zig:93-141, docs/core/api.md:10-12). No compute
call is made here."""
import ctypes as C
import os
import re

import pytest

import turboexl3_b200 as t3
from turboexl3_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE = 0x1000  # a non-null pointer the library must never dereference on a refusal


def declared_functions():
    text = open(os.path.join(ROOT, "include", "t3.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(t3_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    L = t3.lib()
    names = declared_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(L, name), name
        assert name in api.SYMBOLS, f"{name} is declared in t3.h but not bound in api.SYMBOLS"
    assert sorted(api.SYMBOLS) == names


def test_status_names_are_the_references():
    want = {1: "BadExl3Shape", 2: "BadExl3Dtype", 3: "Exl3EngineNotImplemented", 4: "Exl3EngineCacheFull",
            5: "Exl3GateUpRateMismatch", 6: "InvalidExl3Clamp", 7: "InvalidTurboexl3Config", 8: "KernelCreateFailed",
            10: "Exl3TopKExceedsReduceBank", 12: "ExpertLayoutUnsupported", 13: "Exl3WindowUnsupported"}
    for code, name in want.items():
        assert t3.status_name(code) == name


def _linear(in_dim=256, out_dim=256, n=64, rows=1, dt=1, cb=0, w=16, x=FAKE):
    return t3.lib().t3_linear(x, dt, rows, FAKE, FAKE, FAKE, in_dim, out_dim, n, api._Decode(cb, w), FAKE, None, 0, None)


def test_linear_refusals():
    name = t3.status_name
    assert name(_linear(in_dim=200)) == "BadExl3Shape"       # not a multiple of 128
    assert name(_linear(out_dim=64)) == "BadExl3Shape"
    assert name(_linear(n=15)) == "BadExl3Shape"             # odd rate (format.zig:98-101)
    assert name(_linear(n=130)) == "BadExl3Shape"
    assert name(_linear(rows=0)) == "BadExl3Shape"
    assert name(_linear(dt=7)) == "BadExl3Dtype"
    assert name(_linear(w=7)) == "Exl3WindowUnsupported"
    assert name(_linear(cb=5)) == "Exl3EngineNotImplemented"
    assert name(_linear(x=None)) == "NullPointer"


def _bank(hidden=256, inter=128, experts=4, ng=64, nu=64, nd=64):
    p = api._Proj(FAKE, FAKE, FAKE)
    return api._Bank(p, p, p, experts, hidden, inter, ng, nu, nd)


def _moe(bank, rows=1, topk=2, dt=1, sdt=0, ws=FAKE, ws_bytes=1 << 30):
    return t3.lib().t3_moe(FAKE, dt, rows, C.byref(bank), FAKE, FAKE, sdt, topk, api._Decode(0, 16), FAKE, ws, ws_bytes,
                           None)


def test_moe_refusals():
    name = t3.status_name
    assert name(_moe(_bank(hidden=200))) == "BadExl3Shape"
    assert name(_moe(_bank(), topk=33)) == "BadExl3Shape"          # src/root.zig:131
    assert name(_moe(_bank(), topk=0)) == "BadExl3Shape"
    assert name(_moe(_bank(nu=48))) == "Exl3GateUpRateMismatch"    # src/root.zig:117
    assert name(_moe(_bank(nd=48))) == "Exl3EngineNotImplemented"  # src/root.zig:841
    assert name(_moe(_bank(), dt=9)) == "BadExl3Dtype"
    assert name(_moe(_bank(), ws_bytes=16)) == "WorkspaceTooSmall"
    L = t3.lib()
    b = _bank()
    for limit in (0, 129, -3):  # src/root.zig:1002
        rc = L.t3_moe_clamped(FAKE, 1, 1, C.byref(b), FAKE, FAKE, 0, 2, api._Decode(0, 16), limit, FAKE, FAKE, 1 << 30,
                              None)
        assert name(rc) == "InvalidExl3Clamp"
    assert t3.status_name(L.t3_admit_topk(33)) == "Exl3TopKExceedsReduceBank"
    assert L.t3_admit_topk(32) == 0
    assert L.t3_uses_prefill_arm(32) == 0 and L.t3_uses_prefill_arm(33) == 1


def test_workspace_sizes():
    L = t3.lib()
    b = _bank(hidden=2048, inter=512)
    assert L.t3_moe_workspace_bytes(4, 10, C.byref(b)) >= 40 * (512 + 2048) * 2
    assert L.t3_linear_workspace_bytes(1, 2048, 2048, 64) == 0
    # prefill rows: the prepared rows; for few rows of a linear with few 128-column CTAs, the K slices' slab as well (two arms,
    # 33..256 and 257..512 rows; the second only where K is long)
    assert L.t3_linear_workspace_bytes(513, 6144, 2048, 64) == 513 * 6144 * 2
    assert L.t3_linear_workspace_bytes(512, 6144, 2048, 64) > 512 * 6144 * 2 + 4 * 16 * 2 * 128 * 128 * 4
    assert L.t3_linear_workspace_bytes(257, 2048, 2048, 64) == 257 * 2048 * 2
    assert L.t3_linear_workspace_bytes(256, 2048, 2048, 64) > 256 * 2048 * 2 + 2 * 16 * 2 * 128 * 128 * 4
    assert L.t3_linear_workspace_bytes(256, 2048, 6144, 64) == 256 * 2048 * 2  # short K, CTAs past one a multiprocessor
    assert L.t3_linear_workspace_bytes(256, 2048, 32768, 64) == 256 * 2048 * 2  # 256 CTAs a row tile: nothing to cut


def test_expert_quant_json():  # src/core/spec.zig:92-160
    base = '{"expert_quant":{"format":"exl3","k":2.5,"codebook":"mcg"'
    assert t3.parse_expert_quant(base + "}}") == {"n": 40, "codebook": t3.MCG, "window_bits": 16}
    assert t3.parse_expert_quant(base + ',"window":16}}')["window_bits"] == 16
    assert t3.parse_expert_quant(base + ',"window":12}}')["window_bits"] == 12
    for bad in (',"window":7}}', ',"window":17}}', ',"window":"12"}}'):
        with pytest.raises(t3.Exl3Error) as e:
            t3.parse_expert_quant(base + bad)
        assert e.value.name == "Exl3WindowUnsupported"
    assert t3.parse_expert_quant('{"a":1,"expert_quant":{"format":"exl3","k":4,"codebook":"mul1"}}')["n"] == 64
    # the block is a TOP-LEVEL field (src/core/spec.zig:38-40): the same text nested deeper, or inside a string, is not it
    good = '{"format":"exl3","k":4,"codebook":"mul1"}'
    for text in ('{"text_config":{"expert_quant":' + good + '}}', '{"note":"\\"expert_quant\\":' + good.replace('"', '\\"') + '"}',
                 '{"expert_quant":"' + good.replace('"', '\\"') + '"}', '[{"expert_quant":' + good + '}]', '{"expert_quant":' + good):
        with pytest.raises(t3.Exl3Error) as e:
            t3.parse_expert_quant(text)
        assert e.value.name == "ExpertLayoutUnsupported", text
    # sub-keys come from the block itself, not from an object nested inside it
    with pytest.raises(t3.Exl3Error):
        t3.parse_expert_quant('{"expert_quant":{"inner":' + good + '}}')
    for bad in ('{}', '{"expert_quant":{"format":"gptq","k":4,"codebook":"mul1"}}',
                '{"expert_quant":{"format":"exl3","k":4.03,"codebook":"mul1"}}',
                '{"expert_quant":{"format":"exl3","k":9,"codebook":"mul1"}}',
                '{"expert_quant":{"format":"exl3","k":4,"codebook":"mul2"}}',
                '{"expert_quant":{"format":"exl3","codebook":"mul1"}}'):
        with pytest.raises(t3.Exl3Error) as e:
            t3.parse_expert_quant(bad)
        assert e.value.name == "ExpertLayoutUnsupported"


def test_trellis_admitted():  # src/core/spec.zig:80-88
    assert t3.trellis_admitted([8, 16, 32, 64], 8, 256, 512, 64)
    assert t3.trellis_admitted([8, 16, 32, 48], 8, 256, 512, 64)       # at or under the config's rate
    assert not t3.trellis_admitted([8, 16, 32, 80], 8, 256, 512, 64)
    assert not t3.trellis_admitted([8, 16, 32], 8, 256, 512, 64)
    assert not t3.trellis_admitted([8, 16, 31, 64], 8, 256, 512, 64)
    assert not t3.trellis_admitted([8, 16, 32, 63], 8, 256, 512, 64)


def test_configure_validates():  # src/core/config.zig:139
    with pytest.raises(t3.Exl3Error) as e:
        t3.configure(dense_split=17)
    assert e.value.name == "InvalidTurboexl3Config"
    with pytest.raises(t3.Exl3Error):
        t3.configure(ring_bytes=100)
    t3.configure()


def test_release_engines_is_a_no_op_on_empty_caches():
    """src/root.zig:1194-1199: releaseEngines empties every cache; on empty ones it does nothing."""
    api.release_engines()
    assert api.engines_held() == {"decode": 0, "dense": 0, "prefill": 0}


def test_launch_plans_name_kernels_and_shapes():
    """The native kernel seam (src/hip/plan.zig): from a shape alone, the kernel symbols after the reference's naming
    pattern, the grid, block, shared bytes and the buffers by role. No GPU is touched."""
    (l,) = t3.plan_linear(1, 2048, 6144, 64)
    assert l["symbol"] == "t3_dense_gemv_mul1_n64_r8" and l["group"] == "dense"
    assert l["grid"][1] == 6144 // 128 and l["grid"][0] == l["cluster"] and l["block"] == 544
    assert 0 < l["shared"] <= 200 * 1024 and l["roles"][:3] == [0, 7, 3]  # x, y, trellis
    prep, gemv = t3.plan_linear(17, 2048, 2048, 36, t3.Decode(t3.MCG))  # past 8 rows: the rows rotated once, then the GEMV
    assert prep["symbol"] == "t3_dense_prep" and prep["grid"][0] == (17 * 16 + 3) // 4 and prep["roles"] == [0, 1, 4]
    assert gemv["symbol"] == "t3_dense_gemv_mcg_n0_r32" and gemv["roles"][0] == 4  # reads xp
    with pytest.raises(t3.Exl3Error, match="Exl3EngineNotImplemented"):
        t3.plan_linear(33, 2048, 2048, 64)
    with pytest.raises(t3.Exl3Error, match="BadExl3Shape"):
        t3.plan_linear(1, 2000, 2048, 64)
    chain = t3.plan_moe(4, 10, 512, 2048, 512, 48)
    assert [c["symbol"] for c in chain] == ["t3_dec_gate_up_mul1_n48_r8", "t3_dec_down_mul1_n48_r8", "t3_dec_merge"]
    assert chain[0]["grid"][1:] == (512 // 128, 40) and chain[1]["grid"][1:] == (2048 // 128, 40)
    assert chain[0]["cluster"] == chain[0]["grid"][0] and chain[2]["cluster"] == 1
    assert len(t3.plan_moe(2, 1, 1, 2048, 512, 48)) == 2  # one slot a row: the down launch stores y, no merge
