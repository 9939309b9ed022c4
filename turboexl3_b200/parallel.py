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
    """Where each of this rank's row-slots goes. Slot s = row * topk + k."""
    order: torch.Tensor        # [S] slot ids grouped by destination rank (stable: ascending slot inside a rank)
    send_counts: list          # row-slots to each rank
    rows_of_sent: torch.Tensor  # [S] the row of each sent slot, in send order
    local_expert: torch.Tensor  # [S] the expert's index on its owner, in send order (int32)


def plan_dispatch(inds: torch.Tensor, experts: int, world: int) -> DispatchPlan:
    """inds [rows, topk] (any int dtype, any device)."""
    per = experts_per_rank(experts, world)
    flat = inds.reshape(-1).to(torch.int64)
    topk = inds.shape[-1]
    dest = torch.div(flat, per, rounding_mode="floor").clamp_(0, world - 1)
    order = torch.sort(dest, stable=True).indices
    counts = torch.bincount(dest, minlength=world).tolist()
    return DispatchPlan(order, counts, torch.div(order, topk, rounding_mode="floor"),
                        (flat[order] % per).to(torch.int32))


def _all_to_all_rows(send: torch.Tensor, send_counts: list, recv_counts: list, group) -> torch.Tensor:
    recv = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    dist.all_to_all_single(recv, send.contiguous(), recv_counts, send_counts, group=group)
    return recv


def ep_moe(x: torch.Tensor, inds: torch.Tensor, scores: torch.Tensor, experts: int,
           expert_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
           merge_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], group=None) -> torch.Tensor:
    """One routed layer, expert-parallel. x [rows, hidden] (this rank's rows), inds/scores [rows, topk] with GLOBAL
    expert ids. expert_fn(x_recv [R, hidden], local_expert [R] int32) -> v [R, hidden]: each received row through one
    local expert. merge_fn(v [rows, topk, hidden], scores) -> y [rows, hidden]. Returns y for this rank's rows."""
    world = dist.get_world_size(group)
    rows, topk = inds.shape
    plan = plan_dispatch(inds, experts, world)
    counts_out = torch.tensor(plan.send_counts, dtype=torch.int64, device=x.device)
    counts_in = torch.empty_like(counts_out)
    dist.all_to_all_single(counts_in, counts_out, group=group)
    recv_counts = counts_in.tolist()
    x_recv = _all_to_all_rows(x[plan.rows_of_sent], plan.send_counts, recv_counts, group)
    e_recv = _all_to_all_rows(plan.local_expert.to(x.device), plan.send_counts, recv_counts, group)
    v_recv = expert_fn(x_recv, e_recv) if x_recv.shape[0] else x_recv.new_empty((0, x.shape[1]))
    v_back = _all_to_all_rows(v_recv, recv_counts, plan.send_counts, group)
    v = torch.empty_like(v_back)
    v[plan.order] = v_back  # back to slot order
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

    def expert_fn(xr: torch.Tensor, er: torch.Tensor) -> torch.Tensor:
        return expert_rows(xr, bank_local, er, dec)

    def merge_fn(v: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
        return api.moe_merge(v.contiguous(), sc.contiguous(), x.dtype, shared)

    return ep_moe(x, inds, scores, experts, expert_fn, merge_fn, group)


# ---- column-sharded dense linears ----------------------------------------------------------------------------------

def column_blocks(out_dim: int, rank: int, world: int) -> tuple:
    """The 128-column blocks [b0, b1) rank `rank` owns (blocks spread as evenly as they go)."""
    nb = out_dim // 128
    return nb * rank // world, nb * (rank + 1) // world


def shard_columns(trellis: torch.Tensor, svh: torch.Tensor, rank: int, world: int):
    """(trellis shard [in/16, cols/16, n] contiguous, svh shard) of a dense linear for rank `rank`."""
    b0, b1 = column_blocks(trellis.shape[1] * 16, rank, world)
    return trellis[:, b0 * 8:b1 * 8, :].contiguous(), svh[b0 * 128:b1 * 128].contiguous()


def gather_columns(y_local: torch.Tensor, out_dim: int, group=None) -> torch.Tensor:
    """All ranks' column shards [rows, cols_r] into y [rows, out_dim] (shards may differ by one block)."""
    world = dist.get_world_size(group)
    rows = y_local.shape[0]
    widths = [128 * (column_blocks(out_dim, r, world)[1] - column_blocks(out_dim, r, world)[0]) for r in range(world)]
    wmax = max(widths)
    padded = y_local if y_local.shape[1] == wmax else torch.nn.functional.pad(y_local, (0, wmax - y_local.shape[1]))
    parts = [torch.empty((rows, wmax), dtype=y_local.dtype, device=y_local.device) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[:, :w] for p, w in zip(parts, widths)], dim=1)


def column_sharded_linear(x: torch.Tensor, trellis_shard: torch.Tensor, suh: torch.Tensor, svh_shard: torch.Tensor,
                          out_dim: int, dec, group=None, linear_fn=None) -> torch.Tensor:
    """y [rows, out_dim] from this rank's column shard; x and suh are replicated."""
    if linear_fn is None:
        from .api import linear as linear_fn
    if trellis_shard.shape[1] == 0:
        y_local = x.new_empty((x.shape[0], 0))
    else:
        y_local = linear_fn(x, trellis_shard, suh, svh_shard, dec)
    return gather_columns(y_local, out_dim, group)
