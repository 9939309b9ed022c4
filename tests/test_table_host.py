"""The quant-plugin table's claim, validation and load refusals, CPU only: the reference's own table tests
(table/config.zig:150-204) restated against include/t3_table.h. No compute call is made."""
import ctypes as C
import os
import re

import numpy as np

import turboexl3_b200 as t3
from turboexl3_b200 import table as tb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TRUNK = '{"format":"exl3","codebook":"mul1","window":16}'
BANK = '{"format":"exl3","k":5,"codebook":"mul1"}'
QWEN = '{"model_type":"qwen4_exp","trunk_quant":' + TRUNK + ',"text_config":{"num_experts_per_tok":8}}'
QWEN_EXPERTS_ONLY = '{"model_type":"qwen4_exp","text_config":{"num_experts_per_tok":8}}'
GLM = '{"model_type":"glm5_next","swiglu_limit":7.0}'


def test_table_symbols_exported_and_members_named_as_the_reference():
    L = t3.lib()
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "t3_table.h")).read(), flags=re.S)
    declared = sorted(set(re.findall(r"\b(t3_table[a-z0-9_]*)\s*\(", text)))
    assert declared == sorted(tb.TABLE_SYMBOLS)
    for name in declared:
        assert hasattr(L, name)
    t = tb.table()
    assert t.name == b"turboexl3"
    members = [f[0] for f in tb.QuantTable._fields_]
    assert members == ["name", "claims", "validate", "bill", "open", "close", "load_tensor", "load_bank", "release",
                       "matmul", "moe", "swiglu"]  # table/table.zig:30-43


def test_claims():  # table/config.zig:150-170
    t = tb.table()
    claim = lambda b, c: t.claims(b.encode(), c.encode())
    assert claim(TRUNK, "{}") == tb.CLAIM_BY_MARKER
    assert claim(BANK, QWEN) == tb.CLAIM_BY_MARKER
    assert claim(BANK, QWEN_EXPERTS_ONLY) == tb.CLAIM_NO
    assert claim(BANK, '{"model_type":"mimo_v2","trunk_quant":' + TRUNK + "}") == tb.CLAIM_NO
    assert claim(BANK, GLM) == tb.CLAIM_NO
    assert claim('{"format":"stq","k":3,"codebook":"std1"}', QWEN) == tb.CLAIM_NO
    assert claim('{"format":"exl3","k":3,"codebook":"pair1"}', QWEN) == tb.CLAIM_NO
    assert claim('{"bits":4,"group_size":64}', QWEN) == tb.CLAIM_NO
    assert claim("{}", "{}") == tb.CLAIM_NO
    assert claim("{", "{}") == tb.CLAIM_NO


def test_validate():  # table/config.zig:172-189
    t = tb.table()
    val = lambda b, c: t.validate(b.encode(), c.encode())
    assert val(TRUNK, "{}").ok and val(BANK, QWEN).ok
    assert val('{"format":"exl3","codebook":"mcg","window":12}', "{}").ok
    for block, cfg, want in [
        ('{"format":"exl3","codebook":"std1"}', "{}", "Exl3CodebookUnsupported"),
        ('{"format":"exl3","window":7}', "{}", "Exl3WindowUnsupported"),
        ('{"format":"exl3","k":1.03,"codebook":"mul1"}', "{}", "Exl3RateUnsupported"),
        ('{"format":"exl3","k":9,"codebook":"mul1"}', "{}", "Exl3RateUnsupported"),
        (BANK, '{"num_experts_per_tok":33}', "Exl3TopKExceedsReduceBank"),
        ('{"bits":4}', "{}", "NotExl3"),
    ]:
        v = val(block, cfg)
        assert not v.ok and v.why == want, (block, v.why)
    assert t.bill(TRUNK.encode(), b"/models/x", 12345) == 12345


def test_open_reads_the_block():  # table/config.zig:191-204
    b = tb.Block('{"format":"exl3","k":2.5,"codebook":"mcg","window":14}')
    assert b.verdict.ok
    b.close()
    bad = tb.Block('{"format":"exl3","k":9,"codebook":"mul1"}')
    assert not bad.verdict.ok and bad.verdict.why == "Exl3RateUnsupported"


def test_load_refusals_before_any_upload():  # table/table.zig:119-172
    trunk = tb.Block(TRUNK)
    bank = tb.Block(BANK)
    t16 = lambda *s: np.zeros(s, np.uint16)
    f16 = lambda *s: np.zeros(s, np.float16)
    v, _ = bank.load_tensor(t16(8, 8, 64), f16(128), f16(128))
    assert v.why == "turboexl3: dense linears load under the trunk_quant block"
    v, _ = trunk.load_bank(t16(2, 8, 8, 80), f16(2, 128), f16(2, 128))
    assert v.why == "turboexl3: routed banks load under the expert_quant block"
    for args, want in [
        ((t16(8, 8), f16(128), f16(128)), "Exl3TrellisGeometry"),
        ((t16(8, 8, 15), f16(128), f16(128)), "Exl3RateUnsupported"),
        ((t16(7, 8, 64), f16(112), f16(128)), "Exl3WidthNotMultipleOf128"),
        ((t16(8, 8, 64), f16(64), f16(128)), "Exl3SideGeometry"),
        ((t16(8, 8, 64), np.zeros(128, np.float32), f16(128)), "Exl3SideDtype"),
    ]:
        v, _ = trunk.load_tensor(*args)
        assert v.kind == tb.VERDICT_UNSUPPORTED and v.why == want, (want, v.why)
    v, _ = trunk.load_tensor(t16(8, 8, 64), f16(128), f16(128), in_dim=256)
    assert v.why == "Exl3TrellisGeometry"
    for args, want in [
        ((t16(2, 8, 8, 96), f16(2, 128), f16(2, 128)), "Exl3TrellisGeometry"),   # above the block's rate (k = 5)
        ((t16(2, 8, 8, 80), f16(2, 64), f16(2, 128)), "Exl3SideGeometry"),
        ((t16(8, 8, 80), f16(2, 128), f16(2, 128)), "Exl3TrellisGeometry"),
    ]:
        v, _ = bank.load_bank(*args)
        assert v.why == want, (want, v.why)
    trunk.close()
    bank.close()


def test_moe_member_always_refuses():  # table/table.zig:203-205
    w = tb.Weight()
    a = tb.Array()
    v = tb.table().moe(C.byref(w), C.byref(a), C.byref(a), C.byref(a), 0, None, C.byref(a))
    assert v.kind == tb.VERDICT_UNSUPPORTED
    assert v.why == "turboexl3: a layer's banks run as one routed SwiGLU (swiglu)"
    v = tb.table().matmul(C.byref(w), C.byref(a), None, C.byref(a))
    assert v.kind == tb.VERDICT_FAILED and v.why == "turboexl3: a weight without its decode"
