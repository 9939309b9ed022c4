"""The kernels' per-lane trellis reader and pair decoders replayed on the CPU (tests/host_emul/lane_emul.cpp compiles
turboexl3_b200/csrc/t3_lane.cuh with g++) against the oracle's unpackTile/decodeTile: the lane plans of the
reference are held to unpackTile the same way (src/core/lane.zig:178-242; on a GPU, src/hip_tests.zig:59-123)."""
import ctypes
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def emul():
    out = os.path.join(HERE, "host_emul", "_build")
    os.makedirs(out, exist_ok=True)
    so = os.path.join(out, "liblane_emul.so")
    srcs = [os.path.join(HERE, "host_emul", "lane_emul.cpp"), os.path.join(ROOT, "oracle", "t3_oracle.c")]
    hdr = os.path.join(ROOT, "turboexl3_b200", "csrc", "t3_lane.cuh")
    newest = max(os.path.getmtime(p) for p in srcs + [hdr])
    if not os.path.exists(so) or os.path.getmtime(so) < newest:
        obj = os.path.join(out, "t3_oracle.o")
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-std=c11", "-c", srcs[1], "-o", obj], check=True)
        subprocess.run(["g++", "-O1", "-ffp-contract=off", "-fPIC", "-shared", "-std=c++17", "-x", "c++", srcs[0],
                        "-x", "none", obj, "-o", so, "-lm", "-pthread"], check=True)
    return ctypes.CDLL(so)


def test_codebooks_every_codeword(emul):
    assert emul.lane_emul_codebooks() == 0


def test_templated_reader_integer_rates(emul):
    assert emul.lane_emul_integer_rates(8) == 0


def test_templated_reader_fractional_rates(emul):
    assert emul.lane_emul_fractional_rates(4) == 0


def test_runtime_reader_every_rate(emul):
    assert emul.lane_emul_any_rate(4) == 0


def test_lane_order(emul):
    assert emul.lane_emul_lane_order() == 0
