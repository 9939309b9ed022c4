"""t3_moe_noalloc: the routed chain for callers that cannot allocate device memory (a host whose pool owns the GPU, a
plugin that is only handed tensors). It must give the same bytes as t3_moe with a caller workspace, call after call,
although every call reuses one built-in scratch array that is never cleared. Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

import turboexl3_b200 as t3
from turboexl3_b200 import api, synth

pytestmark = pytest.mark.gpu

SCRATCH_LIMIT = 4 << 20


def _bank(seed, experts, hidden, inter, n):
    arrs = synth.bank(seed, experts, hidden, inter, n)
    d = {k: torch.from_numpy(v).cuda() for k, v in arrs.items()}
    return t3.Bank(t3.Proj(d["gate_t"], d["gate_suh"], d["gate_svh"]), t3.Proj(d["up_t"], d["up_suh"], d["up_svh"]),
                   t3.Proj(d["down_t"], d["down_suh"], d["down_svh"]))


def _noalloc(x, bank, inds, scores, dec=t3.Decode.mul1):
    """The new entry point, straight through the C ABI: no workspace argument, no allocation on its behalf."""
    rows, hidden, topk = x.shape[1], x.shape[2], inds.shape[2]
    y = torch.empty_like(x)
    cb = api._bank_c(bank, hidden)
    rc = t3.lib().t3_moe_noalloc(x.data_ptr(), 1, rows, C.byref(cb), inds.data_ptr(), scores.data_ptr(), 0, topk,
                                 dec._c(), y.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, y


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    H, I, E, topk, n = 512, 256, 12, 4, 64
    bank = _bank(91, E, H, I, n)
    bits = lambda t: t.cpu().contiguous().view(torch.int16).numpy()
    # two different calls back to back: the second starts from the first one's leftovers in the shared scratch
    for call, rows in enumerate((16, 3)):
        inds, scores = synth.routing(92 + call, rows, E, topk)
        x = torch.from_numpy(synth.activations(93 + call, rows, H)).cuda().view(1, rows, H)
        di = torch.from_numpy(inds).cuda().view(1, rows, topk)
        ds = torch.from_numpy(scores).cuda().view(1, rows, topk)
        want = t3.moe(x, bank, di, ds)               # the existing entry point, caller-allocated workspace
        rc, got = _noalloc(x, bank, di, ds)
        assert rc == 0, t3.status_name(rc)
        torch.cuda.synchronize()
        assert np.array_equal(bits(got), bits(want)), (call, rows)  # same kernels, same inputs: the same bytes
    assert t3.device_error() == 0


def test_a_warm_call_takes_no_device_memory():
    """The point of the entry: no allocation on the caller's behalf. After a first call (which looks up the scratch array's
    address once), further calls leave the device's free memory where it was and launch the chain's three kernels."""
    H, I, E, topk, n, rows = 512, 256, 12, 4, 64, 8
    bank = _bank(96, E, H, I, n)
    inds, scores = synth.routing(97, rows, E, topk)
    x = torch.from_numpy(synth.activations(98, rows, H)).cuda().view(1, rows, H)
    di = torch.from_numpy(inds).cuda().view(1, rows, topk)
    ds = torch.from_numpy(scores).cuda().view(1, rows, topk)
    y = torch.empty_like(x)
    cb = api._bank_c(bank, H)
    call = lambda: t3.lib().t3_moe_noalloc(x.data_ptr(), 1, rows, C.byref(cb), di.data_ptr(), ds.data_ptr(), 0, topk,
                                           t3.Decode.mul1._c(), y.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert call() == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    launches_before = t3.launch_count()
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert t3.launch_count() - launches_before == 3 * 3  # gate|up, down, merge


def test_sizes_past_the_built_in_scratch_are_refused():
    H, I, E, topk, n = 2048, 512, 4, 32, 32
    bank = _bank(95, E, H, I, n)
    cb = api._bank_c(bank, H)
    assert t3.lib().t3_moe_workspace_bytes(32, topk, C.byref(cb)) > SCRATCH_LIMIT
    x = torch.zeros((1, 32, H), dtype=torch.float16, device="cuda")
    inds = torch.zeros((1, 32, topk), dtype=torch.int32, device="cuda")
    scores = torch.zeros((1, 32, topk), dtype=torch.float32, device="cuda")
    rc, _ = _noalloc(x, bank, inds, scores)
    assert t3.status_name(rc) == "ScratchLimitExceeded"
    x40 = torch.zeros((1, 40, H), dtype=torch.float16, device="cuda")
    i40 = torch.zeros((1, 40, 1), dtype=torch.int32, device="cuda")
    s40 = torch.zeros((1, 40, 1), dtype=torch.float32, device="cuda")
    rc, _ = _noalloc(x40, bank, i40, s40)  # prefill rows need far more scratch than the array holds
    assert t3.status_name(rc) == "ScratchLimitExceeded"
