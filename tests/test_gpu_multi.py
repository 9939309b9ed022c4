"""The sharded paths on two real GPUs over NCCL (skipped with fewer): the expert-parallel routed layer and a
column-sharded trunk linear, each against the single-GPU engine and the oracle. Ranks are child processes; every
collective runs between steps (nothing here waits on a peer from inside a kernel)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, fail):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist

        import turboexl3_b200 as t3
        from oracle import binding as ob
        from turboexl3_b200 import parallel as par
        from turboexl3_b200 import synth
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()

        # ---- expert-parallel routed layer: every rank brings its own rows
        H, I, E, topk, n = 512, 256, 8 * world, 4, 64
        arrs = synth.bank(11, E, H, I, n)
        d = {k: dev(v) for k, v in arrs.items()}
        bank = t3.Bank(t3.Proj(d["gate_t"], d["gate_suh"], d["gate_svh"]), t3.Proj(d["up_t"], d["up_suh"], d["up_svh"]),
                       t3.Proj(d["down_t"], d["down_suh"], d["down_svh"]))
        obank = ob.Bank(E, H, I, n, *[arrs[k] for k in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh", "up_svh",
                                                         "down_t", "down_suh", "down_svh")])
        for rows in (3 + rank, 40 + 7 * rank):  # the owners see decode-row and prefill-row batches
            inds, scores = synth.routing(20 + rank + rows, rows, E, topk)
            x16 = synth.activations(30 + rank + rows, rows, H)
            y = par.ep_moe_cuda(dev(x16), par.local_bank(bank, rank, world), dev(inds), dev(scores), E, t3.Decode.mul1)
            ref = ob.moe_rows(obank, x16.astype(np.float32), inds, scores)
            got = y.float().cpu().numpy()
            assert ob.compare(got, ref, 2.0 ** -11)["max_ratio"] <= 4e-3, f"rank {rank} rows {rows}: EP layer off the oracle"
            one = t3.moe(dev(x16).view(1, rows, H), bank, dev(inds).view(1, rows, topk), dev(scores).view(1, rows, topk))
            assert ob.compare(got, one.float().cpu().numpy().reshape(rows, H), 2.0 ** -11)["max_ratio"] <= 4e-3

        # ---- column-sharded trunk linear: same x everywhere, each rank its 128-column blocks, all-gather
        in_dim, out_dim, k = 1024, 128 * 7, 4
        trellis, suh, svh = synth.linear(41, in_dim, out_dim, 16 * k, scaled=True)
        for rows in (1, 48):
            x = dev(synth.activations(42 + rows, rows, in_dim))
            t_sh, svh_sh = par.shard_columns(dev(trellis), dev(svh), rank, world)
            y = par.column_sharded_linear(x, t_sh, dev(suh), svh_sh, out_dim, t3.Decode.mul1)
            whole = t3.linear(x, dev(trellis), dev(suh), dev(svh))
            # a rank computes whole output columns; at this geometry shard and whole take the same K split (1024 inputs
            # cap it): the same bytes as the single-GPU call
            assert torch.equal(y.view(torch.int16), whole.view(torch.int16)), f"rank {rank} rows {rows}: column shards differ"
            # left sharded (no collective) and gathered as stacked shards: the same columns
            b0, b1 = par.column_blocks(out_dim, rank, world)
            mine = par.column_sharded_linear(x, t_sh, dev(suh), svh_sh, out_dim, t3.Decode.mul1, gather="none")
            assert torch.equal(mine, whole[:, b0 * 128:b1 * 128])
            stacked = par.column_sharded_linear(x, t_sh, dev(suh), svh_sh, out_dim, t3.Decode.mul1, gather="stacked")
            for r in range(world):
                c0, c1 = par.column_blocks(out_dim, r, world)
                assert torch.equal(stacked[r][:, :(c1 - c0) * 128], whole[:, c0 * 128:c1 * 128])
        assert t3.device_error() == 0
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:
        fail.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


def test_two_gpus_ep_layer_and_column_shards():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    fail, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    errors = []
    while not fail.empty():
        errors.append(fail.get())
    assert not errors, errors
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
