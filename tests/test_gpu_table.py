"""The quant-plugin table end to end on host arrays: load once, then `matmul` / `swiglu` with numpy inputs and outputs
(host -> device -> host inside the call), against the oracle; the same through device arrays must give the same bytes."""
import ctypes as C

import numpy as np
import pytest
import torch

import turboexl3_b200 as t3
from oracle import binding as ob
from turboexl3_b200 import synth
from turboexl3_b200 import table as tb

pytestmark = pytest.mark.gpu

TRUNK = '{"format":"exl3","codebook":"mul1","window":16}'


def test_matmul_host_arrays_decode_and_prefill_rows():
    in_dim, out_dim, n = 2048, 512, 64
    trellis, suh, svh = synth.linear(61, in_dim, out_dim, n, scaled=True)
    blk = tb.Block(TRUNK)
    v, w = blk.load_tensor(trellis, suh, svh, in_dim)
    assert v.ok and (w.in_dim, w.out_dim, w.block, w.layout, w.flags) == (in_dim, out_dim, n, 0, 16)
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, ob.MUL1)
    for rows in (1, 5, 32, 70):
        x = synth.activations(62 + rows, rows, in_dim)
        v, y = tb.matmul(w, x)
        assert v.ok, v.why
        ref = ob.linear_rows_what(x.astype(np.float32), what, suh, svh, in_dim, out_dim)
        assert ob.compare(y.astype(np.float32), ref)["max_ratio"] <= 5e-3
        # device arrays: no staging, same bytes
        xd = torch.from_numpy(x).cuda()
        yd = torch.empty((rows, out_dim), dtype=torch.float16, device="cuda")
        out = tb.device_array(yd.data_ptr(), 1, (rows, out_dim))
        v = tb.table().matmul(C.byref(w), C.byref(tb.device_array(xd.data_ptr(), 1, (rows, in_dim))),
                              torch.cuda.current_stream().cuda_stream, C.byref(out))
        assert v.ok
        assert np.array_equal(yd.cpu().numpy().view(np.uint16), y.view(np.uint16))
    x3 = synth.activations(99, 6, in_dim).reshape(2, 3, in_dim)
    v, y3 = tb.matmul(w, x3)
    assert v.ok and y3.shape == (2, 3, out_dim)
    v, _ = tb.matmul(w, np.zeros((2, in_dim + 128), np.float16))
    assert v.why == "BadExl3Shape"
    assert tb.table().release(C.byref(w)) is None and w.w is None
    blk.close()
    assert t3.lib().t3_table_staging_bytes() > 0
    t3.lib().t3_table_release_staging()
    assert t3.lib().t3_table_staging_bytes() == 0


def test_swiglu_host_arrays():
    H, I, E, topk, n = 512, 256, 8, 4, 48
    arrs = synth.bank(71, E, H, I, n)
    blk = tb.Block('{"format":"exl3","k":3,"codebook":"mul1"}')
    ws = {}
    for name in ("gate", "up", "down"):
        v, ws[name] = blk.load_bank(arrs[name + "_t"], arrs[name + "_suh"], arrs[name + "_svh"])
        assert v.ok, v.why
    obank = ob.Bank(E, H, I, n, *[arrs[k] for k in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh", "up_svh",
                                                     "down_t", "down_suh", "down_svh")])
    for rows in (1, 4, 48):
        inds, scores = synth.routing(72 + rows, rows, E, topk)
        x = synth.activations(73 + rows, rows, H).reshape(1, rows, H)
        v, y = tb.swiglu(ws["gate"], ws["up"], ws["down"], x, inds.reshape(1, rows, topk), scores.reshape(1, rows, topk))
        assert v.ok, v.why
        ref = ob.moe_rows(obank, x.reshape(rows, H).astype(np.float32), inds, scores)
        assert ob.compare(y.reshape(rows, H).astype(np.float32), ref)["max_ratio"] <= 5e-3
    # the clamped call (opts.limit > 0) runs moeClamped; a limit past 128 is refused by name
    inds, scores = synth.routing(5, 2, E, topk)
    x = synth.activations(6, 2, H).reshape(1, 2, H)
    v, y = tb.swiglu(ws["gate"], ws["up"], ws["down"], x, inds.reshape(1, 2, topk), scores.reshape(1, 2, topk), limit=1)
    ref = ob.moe_rows(obank, x.reshape(2, H).astype(np.float32), inds, scores, limit=1.0)
    assert v.ok and ob.compare(y.reshape(2, H).astype(np.float32), ref)["max_ratio"] <= 5e-3
    v, _ = tb.swiglu(ws["gate"], ws["up"], ws["down"], x, inds.reshape(1, 2, topk), scores.reshape(1, 2, topk), limit=129)
    assert v.why == "InvalidExl3Clamp"
    for w in ws.values():
        tb.table().release(C.byref(w))
    blk.close()
    assert t3.device_error() == 0


def test_device_array_calls_on_two_streams_do_not_share_scratch():
    """Calls on device arrays return with their kernels in flight; two such calls on two streams run at once. Each stream has
    its own workspace in the table, so the results are the serial ones."""
    H, I, E, topk, n, rows = 512, 256, 8, 4, 48, 64
    arrs = synth.bank(75, E, H, I, n)
    blk = tb.Block('{"format":"exl3","k":3,"codebook":"mul1"}')
    ws = {}
    for name in ("gate", "up", "down"):
        v, ws[name] = blk.load_bank(arrs[name + "_t"], arrs[name + "_suh"], arrs[name + "_svh"])
        assert v.ok, v.why
    tab = tb.table()
    calls = []
    for c in range(2):
        inds, scores = synth.routing(76 + c, rows, E, topk)
        x = torch.from_numpy(synth.activations(77 + c, rows, H)).cuda()
        di, ds = torch.from_numpy(inds).cuda(), torch.from_numpy(scores).cuda()
        y = torch.zeros((rows, H), dtype=torch.float16, device="cuda")
        calls.append((x, di, ds, y))

    def run(call, stream):
        x, di, ds, y = call
        out = tb.device_array(y.data_ptr(), 1, (1, rows, H))
        v = tab.swiglu(C.byref(ws["gate"]), C.byref(ws["up"]), C.byref(ws["down"]),
                       C.byref(tb.device_array(x.data_ptr(), 1, (1, rows, H))),
                       C.byref(tb.device_array(di.data_ptr(), 5, (1, rows, topk))),
                       C.byref(tb.device_array(ds.data_ptr(), 0, (1, rows, topk))), C.byref(tb.SwigluOpts(0, 0)),
                       stream.cuda_stream, C.byref(out))
        assert v.ok, v.why

    main = torch.cuda.current_stream()
    serial = []
    for call in calls:
        run(call, main)
        torch.cuda.synchronize()
        serial.append(call[3].clone())
        call[3].zero_()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for s in streams:
        s.wait_stream(main)
    for _ in range(4):  # several rounds, both streams busy at once
        for call, s in zip(calls, streams):
            run(call, s)
    torch.cuda.synchronize()
    for call, want in zip(calls, serial):
        assert torch.equal(call[3], want)
    for w in ws.values():
        tab.release(C.byref(w))
    blk.close()
    assert t3.device_error() == 0


def test_pack_file_to_table_to_matmul(tmp_path):
    """A trunk linear from a safetensors shard (the reference's affine names, i16 trellis) through the table's loader."""
    from turboexl3_b200 import pack
    in_dim, out_dim, n = 512, 256, 80
    trellis, suh, svh = synth.linear(81, in_dim, out_dim, n, scaled=True)
    pack.write_safetensors(str(tmp_path / "shard.safetensors"),
                           {"attn.o.weight": trellis.view(np.int16), "attn.o.scales": suh, "attn.o.biases": svh})
    pk = pack.Pack.open_dir(str(tmp_path))
    blk = tb.Block(TRUNK)
    v, w = blk.load_tensor(*pk.trunk("attn.o"), in_dim)
    assert v.ok, v.why
    x = synth.activations(82, 9, in_dim)
    v, y = tb.matmul(w, x)
    assert v.ok
    want = t3.linear(torch.from_numpy(x).cuda(), torch.from_numpy(trellis).cuda(), torch.from_numpy(suh).cuda(),
                     torch.from_numpy(svh).cuda())
    assert np.array_equal(y.view(np.uint16), want.cpu().numpy().view(np.uint16))
    tb.table().release(C.byref(w))
    blk.close()
    pk.close()
