"""The multi-GPU sharding of the path on CPU ranks (gloo, world size 2 and 3): the dispatch plan, the two all-to-alls of
the expert-parallel layer and the column-shard gather, with stand-in compute functions. No GPU, no kernels: the index
arithmetic of turboexl3_b200/parallel.py is what is under test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from turboexl3_b200 import parallel as par


def test_plan_dispatch_groups_slots_by_owner_in_slot_order():
    inds = torch.tensor([[5, 0, 3], [1, 7, 2]], dtype=torch.int32)  # 8 experts over 4 ranks: 2 each
    plan = par.plan_dispatch(inds, 8, 4)
    assert plan.send_counts == [2, 2, 1, 1]
    assert plan.order.tolist() == [1, 3, 2, 5, 0, 4]          # dest 0: slots 1,3; dest 1: 2,5; dest 2: 0; dest 3: 4
    assert plan.rows_of_sent.tolist() == [0, 1, 0, 1, 0, 1]
    assert plan.local_expert.tolist() == [0, 1, 1, 0, 1, 1]
    # a row travels once to each rank that owns any of its experts; each sent slot names its row inside that rank's group
    assert plan.row_counts == [2, 2, 1, 1] and plan.send_rows.tolist() == [0, 1, 0, 1, 0, 1]
    assert plan.row_in_group.tolist() == [0, 1, 0, 1, 0, 0]
    dup = par.plan_dispatch(torch.tensor([[0, 1, 4], [5, 2, 3]], dtype=torch.int32), 8, 2)  # 4 experts a rank
    assert dup.send_counts == [4, 2] and dup.row_counts == [2, 2]       # row 0 -> rank 0 twice, once to rank 1: sent once each
    assert dup.send_rows.tolist() == [0, 1, 0, 1] and dup.row_in_group.tolist() == [0, 0, 1, 1, 0, 1]
    with pytest.raises(ValueError):
        par.plan_dispatch(inds, 7, 4)


def test_column_blocks_cover_every_block_once():
    for out_dim, world in ((7168, 8), (2048, 8), (640, 4), (24576, 8), (128, 2)):
        spans = [par.column_blocks(out_dim, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == out_dim // 128
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, fail):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        experts, hidden, topk = 6 * world, 16, 3
        per = experts // world
        g = torch.Generator().manual_seed(100 + rank)
        rows = [5, 0, 3][rank % 3] if world > 1 else 4       # one rank has no rows at all
        x = torch.randn((rows, hidden), generator=g)
        inds = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(rows)]).to(torch.int32) \
            if rows else torch.zeros((0, topk), dtype=torch.int32)
        if rank == 0 and rows:
            inds[:, :] = inds % per                           # rank 0 sends everything to itself and receives from others
        scores = torch.rand((rows, topk), generator=g)

        def expert_fn(xr, row_of_slot, er):                   # stand-in expert: scales by (global expert id + 1)
            return xr[row_of_slot.to(torch.int64)] * (er.to(torch.float32) + 1.0 + rank * per).unsqueeze(1)

        def merge_fn(v, sc):
            y = torch.zeros((v.shape[0], v.shape[2]))
            for k in range(v.shape[1]):                       # slot order
                y = y + sc[:, k:k + 1] * v[:, k]
            return y

        y = par.ep_moe(x, inds, scores, experts, expert_fn, merge_fn)
        want = merge_fn(x.unsqueeze(1) * (inds.to(torch.float32) + 1.0).unsqueeze(2), scores)
        assert y.shape == want.shape and torch.equal(y, want), f"rank {rank}: ep_moe differs"

        # column-sharded linear: a stand-in linear whose output column c is x[:, 0] * svh[c] + number of its tiles' rows
        in_dim, out_dim, n = 256, 128 * 5, 16                # 5 blocks: uneven over 2 or 3 ranks
        gw = torch.Generator().manual_seed(7)
        trellis = torch.randint(0, 2 ** 15, (in_dim // 16, out_dim // 16, n), generator=gw, dtype=torch.int16)
        svh = torch.randn(out_dim, generator=gw).to(torch.float16)
        suh = torch.ones(in_dim, dtype=torch.float16)
        xs = torch.randn((4, in_dim), generator=gw)

        def fake_linear(xx, tr, su, sv, dec):
            col_sig = tr.to(torch.float32).sum(dim=(0, 2)).repeat_interleave(16)  # one value a tile column: identifies the shard
            return xx[:, :1] * sv.to(torch.float32)[None, :] + col_sig[None, :]

        t_shard, svh_shard = par.shard_columns(trellis, svh, rank, world)
        y = par.column_sharded_linear(xs, t_shard, suh, svh_shard, out_dim, None, linear_fn=fake_linear)
        assert torch.equal(y, fake_linear(xs, trellis, suh, svh, None)), f"rank {rank}: gathered columns differ"
        stacked = par.column_sharded_linear(xs, t_shard, suh, svh_shard, out_dim, None, linear_fn=fake_linear, gather="stacked")
        b0, b1 = par.column_blocks(out_dim, rank, world)
        assert stacked.shape[0] == world and torch.equal(stacked[rank][:, :128 * (b1 - b0)], y[:, 128 * b0:128 * b1])
        mine = par.column_sharded_linear(xs, t_shard, suh, svh_shard, out_dim, None, linear_fn=fake_linear, gather="none")
        assert torch.equal(mine, y[:, 128 * b0:128 * b1])
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # surface the failure in the parent
        fail.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


@pytest.mark.parametrize("world", [2, 3])
def test_ep_and_column_shards_on_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    fail = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    errors = []
    while not fail.empty():
        errors.append(fail.get())
    assert not errors, errors
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def test_mixed_rate_buckets_route_every_slot_to_its_sub_bank():
    """The mixed-rate layer's index arithmetic with host stand-ins for the engine: expert e scales its row by e + 1."""
    from turboexl3_b200 import mixed
    g = torch.Generator().manual_seed(5)
    E, rows, topk, H = 11, 9, 3, 8
    rates = [32, 48, 64, 48, 32, 32, 64, 48, 48, 64, 32]
    b = mixed.bucket_by_rate(rates)
    assert b.rates == [32, 48, 64]
    assert b.members == [[0, 4, 5, 10], [1, 3, 7, 8], [2, 6, 9]]
    for e in range(E):
        assert b.members[int(b.bank_of[e])][int(b.local_of[e])] == e
    x = torch.randn(rows, H, generator=g).half()
    inds = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(rows)]).to(torch.int32)
    scores = torch.rand(rows, topk, generator=g)
    banks = [torch.tensor(m) for m in b.members]  # a "bank" here is just its experts' ids
    expert_fn = lambda xr, bank, er: (xr.float() * (bank[er.long()].float() + 1.0).unsqueeze(1)).half()
    merge_fn = lambda v, sc: (v.float() * sc.unsqueeze(-1)).sum(1)
    y = mixed.mixed_rate_moe(x, banks, b, inds, scores, None, expert_fn=expert_fn, merge_fn=merge_fn)
    want = ((x.float().unsqueeze(1) * (inds.float() + 1.0).unsqueeze(-1)).half().float() * scores.unsqueeze(-1)).sum(1)
    assert torch.allclose(y, want, rtol=0, atol=1e-6)
