"""The safetensors pack reader (host side): round trip, the reference's tensor names, refusals, and the hand-over to
the plugin table's loaders (validation only: no GPU)."""
import json
import struct

import numpy as np
import pytest

from turboexl3_b200 import pack, synth


def test_round_trip_names_and_views(tmp_path):
    trellis, suh, svh = synth.linear(1, 256, 128, 48)
    arrs = synth.bank(2, 3, 256, 128, 32)
    p1, p2 = tmp_path / "a.safetensors", tmp_path / "b.safetensors"
    pack.write_safetensors(str(p1), {"model.q.weight": trellis.view(np.int16), "model.q.scales": suh, "model.q.biases": svh},
                           {"format": "exl3"})
    pack.write_safetensors(str(p2), {"mlp.gate.trellis": arrs["gate_t"], "mlp.gate.suh": arrs["gate_suh"],
                                     "mlp.gate.svh": arrs["gate_svh"]})
    pk = pack.Pack.open_dir(str(tmp_path))
    t, a, b = pk.trunk("model.q")
    assert t.dtype == np.uint16 and np.array_equal(t, trellis) and np.array_equal(a, suh) and np.array_equal(b, svh)
    bt, ba, bb = pk.bank("mlp.gate")
    assert bt.shape == (3, 16, 8, 32) and np.array_equal(bt, arrs["gate_t"]) and np.array_equal(bb, arrs["gate_svh"])
    assert not t.flags.writeable  # a view of the mapping, not a copy
    assert pk.shards[0].metadata == {"format": "exl3"}
    with pytest.raises(pack.PackError, match="MissingWeight"):
        pk.trunk("model.k")
    del t, a, b, bt, ba, bb
    pk.close()


def test_malformed_files_are_refused(tmp_path):
    short = tmp_path / "short.safetensors"
    short.write_bytes(b"\x01\x02")
    with pytest.raises(pack.PackError):
        pack.Shard(str(short))
    long_header = tmp_path / "long.safetensors"
    long_header.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(pack.PackError):
        pack.Shard(str(long_header))
    hdr = json.dumps({"w": {"dtype": "F16", "shape": [4], "data_offsets": [0, 64]}}).encode()
    outside = tmp_path / "outside.safetensors"
    outside.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(pack.PackError):
        pack.Shard(str(outside))
    hdr = json.dumps({"w": {"dtype": "F16", "shape": [5], "data_offsets": [0, 8]}}).encode()
    wrong = tmp_path / "wrong.safetensors"
    wrong.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    sh = pack.Shard(str(wrong))
    with pytest.raises(pack.PackError):
        sh.tensor("w")
    sh.close()
