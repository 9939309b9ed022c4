"""Sharding the path over the GPUs of one box: one process a GPU, torch.distributed for the exchange.

The reference runs on a single device and has no counterpart to this file. The path shards two ways:

* Routed experts, expert-parallel: rank r holds experts [r E/G, (r+1) E/G) whole. Every rank routes its own rows: each
  row-slot's activation row goes to the expert's owner (all-to-all "dispatch"), the owner runs its experts on what it
  received (top-1, score 1: the finished down projection `v`, f16), the `v` rows travel back (all-to-all "combine"), and
  the home rank does the score-weighted sum in slot order (`t3.moe_merge`). The weighted sum happens at home in the same
  order whatever G is, so the result does not depend on the number of ranks beyond the kernels' own path choice
  (decode-row chain up to 32 received rows, prefill chain past that).
* Dense trunk linears, column-sharded at 128-column granularity: the output rotation and svh are per 128-output block and
  the input rotation depends on x only, so a rank computes complete output columns with no partial sums; shards are
  gathered with an all-gather.

The exchange steps take injectable compute functions so their index arithmetic runs on CPU ranks (gloo) in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


# ---- expert-parallel routed experts --------------------------------------------------------------------------------

def experts_per_rank(experts: int, world: int) -> int:
    if experts % world:
        raise ValueError(f"{experts} experts do not divide over {world} ranks")
    return experts // world


@dataclass
class DispatchPlan:
    """Where each of this rank's row-slots goes. Slot s = row * topk + k. A token row travels ONCE to every rank that owns
    any of its experts (not once per slot): `send_rows` lists the rows to send grouped by destination, and every sent slot
    names its row by position inside its destination's group."""
    order: torch.Tensor        # [S] slot ids grouped by destination rank (stable: ascending slot inside a rank)
    send_counts: list          # row-slots to each rank
    rows_of_sent: torch.Tensor  # [S] the row of each sent slot, in send order
    local_expert: torch.Tensor  # [S] the expert's index on its owner, in send order (int32)
    send_rows: torch.Tensor     # [R] distinct (destination, row) pairs' rows, grouped by destination, rows ascending
    row_counts: list           # token rows to each rank
    row_in_group: torch.Tensor  # [S] for each sent slot, the position of its row inside its destination's group (int32)
    where: Optional[torch.Tensor] = None   # [S] slot s's position in send order (order's inverse), when the planner gives it
    meta: Optional[torch.Tensor] = None    # [S, 2] int32 (row_in_group, local_expert) already interleaved
    counts_dev: Optional[torch.Tensor] = None  # [2, world] int32 on the device: (send_counts, row_counts)


def plan_dispatch(inds: torch.Tensor, experts: int, world: int) -> DispatchPlan:
    """inds [rows, topk] (any int dtype, any device). One host read: the per-destination counts."""
    per = experts_per_rank(experts, world)
    flat = inds.reshape(-1).to(torch.int64)
    rows, topk = inds.shape
    dest = torch.div(flat, per, rounding_mode="floor").clamp_(0, world - 1)
    order = torch.sort(dest, stable=True).indices
    rows_of_sent = torch.div(order, topk, rounding_mode="floor")
    dest_sent = dest[order]
    # the (destination, row) pairs in send order are already sorted (stable sort, slots of a row are adjacent): distinct
    # pairs are runs
    key = dest_sent * max(rows, 1) + rows_of_sent
    uniq, inverse = torch.unique_consecutive(key, return_inverse=True)
    row_dest = torch.div(uniq, max(rows, 1), rounding_mode="floor")
    slot_counts = torch.bincount(dest, minlength=world)
    row_counts = torch.bincount(row_dest, minlength=world)
    starts = torch.cumsum(row_counts, 0) - row_counts
    counts = torch.stack([slot_counts, row_counts]).tolist()  # the plan's one host read
    return DispatchPlan(order, counts[0], rows_of_sent, (flat[order] % per).to(torch.int32), uniq % max(rows, 1), counts[1],
                        (inverse - starts[dest_sent]).to(torch.int32))


def _all_to_all_rows(send: torch.Tensor, send_counts: list, recv_counts: list, group) -> torch.Tensor:
    if dist.get_world_size(group) == 1:
        return send  # a world of one: what is sent is what is received
    recv = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    dist.all_to_all_single(recv, send.contiguous(), recv_counts, send_counts, group=group)
    return recv


def ep_moe(x: torch.Tensor, inds: torch.Tensor, scores: torch.Tensor, experts: int,
           expert_fn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
           merge_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], group=None,
           plan_fn: Optional[Callable] = None, mapped_merge_fn: Optional[Callable] = None) -> torch.Tensor:
    """One routed layer, expert-parallel. x [rows, hidden] (this rank's rows), inds/scores [rows, topk] with GLOBAL
    expert ids. expert_fn(x_recv [R, hidden], row_of_slot [S] int32, local_expert [S] int32) -> v [S, hidden]: received
    slot i runs row x_recv[row_of_slot[i]] through local expert local_expert[i]. merge_fn(v [rows, topk, hidden], scores)
    -> y [rows, hidden]; or mapped_merge_fn(v_back [S, hidden] in send order, where [S], scores) when the planner gives
    `where` (no reordering copy of v). plan_fn(inds, experts, world) -> DispatchPlan (default: `plan_dispatch`, torch ops).
    Returns y for this rank's rows.

    Exchanges: the counts (one small all-to-all; the plan's counts and the received counts are the two host reads), the
    distinct token rows, the per-slot (row, expert) pairs, and the finished per-slot outputs back."""
    world = dist.get_world_size(group)
    rows, topk = inds.shape
    plan = (plan_fn or plan_dispatch)(inds, experts, world)
    if plan.counts_dev is not None:
        counts_out = plan.counts_dev.t().contiguous()
    else:
        counts_out = torch.tensor([plan.send_counts, plan.row_counts], dtype=torch.int32, device=x.device).t().contiguous()
    if world == 1:
        recv_slots, recv_rows = plan.send_counts, plan.row_counts
    else:
        counts_in = torch.empty_like(counts_out)
        dist.all_to_all_single(counts_in, counts_out, group=group)
        recv = counts_in.t().tolist()
        recv_slots, recv_rows = recv[0], recv[1]
    x_recv = _all_to_all_rows(x[plan.send_rows], plan.row_counts, recv_rows, group)
    meta = plan.meta if plan.meta is not None else torch.stack([plan.row_in_group.to(x.device), plan.local_expert.to(x.device)], dim=1)
    meta_recv = _all_to_all_rows(meta, plan.send_counts, recv_slots, group)  # [S, 2] int32
    row_of_slot = meta_recv[:, 0]
    if world > 1:
        # a received slot names its row inside its SOURCE's group: shift by where that source's rows start here
        starts = [sum(recv_rows[:r]) for r in range(world)]
        shift = torch.repeat_interleave(torch.tensor(starts, dtype=torch.int32, device=x.device),
                                        torch.tensor(recv_slots, device=x.device), output_size=sum(recv_slots))
        row_of_slot = row_of_slot + shift
    if meta_recv.shape[0]:
        v_recv = expert_fn(x_recv, row_of_slot.contiguous(), meta_recv[:, 1].contiguous())
    else:
        v_recv = x_recv.new_empty((0, x.shape[1]))
    v_back = _all_to_all_rows(v_recv, recv_slots, plan.send_counts, group)
    if mapped_merge_fn is not None and plan.where is not None:
        return mapped_merge_fn(v_back, plan.where, scores)
    v = torch.empty_like(v_back)
    v[plan.order.to(torch.int64)] = v_back  # back to slot order
    return merge_fn(v.view(rows, topk, x.shape[1]), scores)


def local_bank(bank, rank: int, world: int):
    """Rank `rank`'s experts of a bank (`turboexl3_b200.Bank` of expert-major tensors): views, no copy."""
    from .api import Bank, Proj
    per = experts_per_rank(bank.gate.trellis.shape[0], world)
    cut = lambda p: Proj(p.trellis[rank * per:(rank + 1) * per], p.suh[rank * per:(rank + 1) * per],
                         p.svh[rank * per:(rank + 1) * per])
    return Bank(cut(bank.gate), cut(bank.up), cut(bank.down))


def ep_moe_cuda(x: torch.Tensor, bank_local, inds: torch.Tensor, scores: torch.Tensor, experts: int, dec,
                shared: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """ep_moe on the engine: x [rows, hidden] on this rank's GPU, bank_local = this rank's experts."""
    from . import api
    from .mixed import expert_rows

    def expert_fn(xr: torch.Tensor, row_of_slot: torch.Tensor, er: torch.Tensor) -> torch.Tensor:
        if er.shape[0] > api.DECODE_ROWS_MAX:
            # the routed prefill chain over gathered rows (root.moeSwigluRows): a row several slots share is read in place
            ones = torch.ones(er.shape[0], dtype=torch.float32, device=xr.device)
            return api.moe_swiglu_rows(xr, row_of_slot, bank_local, er, ones, dec, out_dtype=torch.float16)
        return expert_rows(xr[row_of_slot.to(torch.int64)], bank_local, er, dec)

    def merge_fn(v: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
        return api.moe_merge(v.contiguous(), sc.contiguous(), x.dtype, shared)

    def mapped_merge_fn(v_back: torch.Tensor, where: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
        return api.moe_merge(v_back.contiguous(), sc.contiguous(), x.dtype, shared, where=where)

    def plan_fn(ids: torch.Tensor, n_experts: int, world: int) -> DispatchPlan:
        # the plan in one launch on the device (t3_ep_plan); its counts are the one host read
        order, where, send_rows, meta, counts = api.ep_plan(ids.to(torch.int32).contiguous(), n_experts, world)
        c = counts.tolist()
        return DispatchPlan(order, c[0], None, meta[:, 1], send_rows[:sum(c[1])], c[1], meta[:, 0], where=where, meta=meta,
                            counts_dev=counts)

    world = dist.get_world_size(group)
    device_plan = world <= api.EP_WORLD_MAX and inds.is_cuda
    return ep_moe(x, inds, scores, experts, expert_fn, merge_fn, group, plan_fn if device_plan else None,
                  mapped_merge_fn if device_plan else None)


# ---- column-sharded dense linears ----------------------------------------------------------------------------------

def column_blocks(out_dim: int, rank: int, world: int) -> tuple:
    """The 128-column blocks [b0, b1) rank `rank` owns (blocks spread as evenly as they go)."""
    nb = out_dim // 128
    return nb * rank // world, nb * (rank + 1) // world


def shard_columns(trellis: torch.Tensor, svh: torch.Tensor, rank: int, world: int):
    """(trellis shard [in/16, cols/16, n] contiguous, svh shard) of a dense linear for rank `rank`."""
    b0, b1 = column_blocks(trellis.shape[1] * 16, rank, world)
    return trellis[:, b0 * 8:b1 * 8, :].contiguous(), svh[b0 * 128:b1 * 128].contiguous()


def gather_columns(y_local: torch.Tensor, out_dim: int, group=None, stacked: bool = False) -> torch.Tensor:
    """All ranks' column shards [rows, cols_r] in one collective (all_gather_into_tensor). stacked=True returns the
    buffer as gathered, [world, rows, cols_max] (a head-parallel consumer reads its shard in place; shards narrower than
    the widest are zero-padded on the right); else y [rows, out_dim] (one more copy: the shards interleaved by row)."""
    world = dist.get_world_size(group)
    rows = y_local.shape[0]
    widths = [128 * (column_blocks(out_dim, r, world)[1] - column_blocks(out_dim, r, world)[0]) for r in range(world)]
    wmax = max(widths)
    padded = y_local if y_local.shape[1] == wmax else torch.nn.functional.pad(y_local, (0, wmax - y_local.shape[1]))
    buf = torch.empty((world, rows, wmax), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(buf.view(world * rows, wmax), padded.contiguous(), group=group)  # rank r's rows at [r]
    if stacked:
        return buf
    if all(w == wmax for w in widths):
        return buf.permute(1, 0, 2).reshape(rows, world * wmax)
    return torch.cat([buf[r, :, :w] for r, w in enumerate(widths)], dim=1)


def column_sharded_linear(x: torch.Tensor, trellis_shard: torch.Tensor, suh: torch.Tensor, svh_shard: torch.Tensor,
                          out_dim: int, dec, group=None, linear_fn=None, gather: str = "full") -> torch.Tensor:
    """y from this rank's column shard; x and suh are replicated. gather: "full" -> y [rows, out_dim] on every rank;
    "stacked" -> [world, rows, cols_max] as gathered; "none" -> this rank's shard [rows, cols_r], no collective (the
    consumer is sharded the same way). (Gathering in row chunks on a second stream beside the GEMM was measured and
    dropped: at 4096 rows four chunks took 1876 us against 439 us for one gather after one GEMM.)"""
    if linear_fn is None:
        from .api import linear as linear_fn
    if trellis_shard.shape[1] == 0:
        y_local = x.new_empty((x.shape[0], 0))
    else:
        y_local = linear_fn(x, trellis_shard, suh, svh_shard, dec)
    if gather == "none":
        return y_local
    return gather_columns(y_local, out_dim, group, stacked=gather == "stacked")
