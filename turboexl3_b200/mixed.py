"""Routed experts whose rates differ from expert to expert.

The reference serves one rate per bank (moe requires gate, up and down of a bank to share n: src/root.zig:841, and a
bank's geometry carries a single rate: src/core/decode.zig Geometry.rate), so a layer whose experts were quantised at
different bit widths is held as one sub-bank per rate. This module routes such a layer: every row-slot goes to the sub-bank
that holds its expert, each sub-bank runs its slots at top-1 with score 1 (the finished down projection `v`, f16, exactly
what the single-bank chain feeds its merge), and the score-weighted sum runs once over all slots in slot order
(`t3.moe_merge`) — so the result is the one a single bank of those experts would give, whatever the bucketing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass
class RateBuckets:
    """Which sub-bank holds each expert and where. bank_of[e] indexes `rates`; local_of[e] is e's index in its sub-bank;
    members[b] lists sub-bank b's experts in sub-bank order (ascending expert id)."""
    rates: list
    bank_of: torch.Tensor
    local_of: torch.Tensor
    members: list


def bucket_by_rate(expert_rates: Sequence[int]) -> RateBuckets:
    """expert_rates[e] = n (halfwords per tile) of expert e. Sub-banks are ordered by ascending rate."""
    rates = sorted(set(int(r) for r in expert_rates))
    bank_of = torch.tensor([rates.index(int(r)) for r in expert_rates], dtype=torch.int64)
    local_of = torch.zeros_like(bank_of)
    members = []
    for b in range(len(rates)):
        ids = torch.nonzero(bank_of == b).flatten()
        local_of[ids] = torch.arange(ids.numel())
        members.append(ids.tolist())
    return RateBuckets(rates, bank_of, local_of, members)


def expert_rows(x_rows: torch.Tensor, bank, local_expert: torch.Tensor, dec) -> torch.Tensor:
    """v [R, hidden] f16: row i of x_rows through expert local_expert[i] of `bank` (top-1, score 1)."""
    from . import api
    if x_rows.dtype == torch.bfloat16:
        x_rows = x_rows.float()  # exact, and an f32 call returns v itself where a bf16 call would round it again
    r = x_rows.shape[0]
    if r == 0:
        return x_rows.new_empty((0, x_rows.shape[1]), dtype=torch.float16)
    ones = torch.ones((1, r, 1), dtype=torch.float32, device=x_rows.device)
    out = []
    for r0 in range(0, r, 1 << 16):  # keep every call's row count inside the engine's limits
        r1 = min(r, r0 + (1 << 16))
        out.append(api.moe(x_rows[r0:r1].unsqueeze(0).contiguous(), bank,
                           local_expert[r0:r1].to(torch.int32).view(1, -1, 1).contiguous(), ones[:, r0:r1].contiguous(),
                           dec).squeeze(0))
    return torch.cat(out).to(torch.float16)


def mixed_rate_moe(x: torch.Tensor, banks: Sequence, buckets: RateBuckets, inds: torch.Tensor, scores: torch.Tensor, dec,
                   shared: Optional[torch.Tensor] = None, expert_fn=None, merge_fn=None) -> torch.Tensor:
    """x [rows, hidden]; banks[b] = the sub-bank of rate buckets.rates[b]; inds/scores [rows, topk] with the layer's
    expert ids. Returns y [rows, hidden] in x's dtype. expert_fn(x_rows, bank, local_expert) -> v and
    merge_fn(v [rows, topk, hidden], scores) -> y default to the engine; tests inject host stand-ins."""
    if expert_fn is None:
        expert_fn = lambda xr, bank, er: expert_rows(xr, bank, er, dec)
    if merge_fn is None:
        from . import api
        merge_fn = lambda vv, sc: api.moe_merge(vv, sc.contiguous(), x.dtype, shared)
    rows, topk = inds.shape
    flat = inds.reshape(-1).to(torch.int64)
    bank_of, local_of = buckets.bank_of.to(flat.device), buckets.local_of.to(flat.device)
    slot_bank = bank_of[flat]
    v = torch.empty((rows * topk, x.shape[1]), dtype=torch.float16, device=x.device)
    for b, bank in enumerate(banks):
        sel = torch.nonzero(slot_bank == b).flatten()
        if sel.numel():
            v[sel] = expert_fn(x[torch.div(sel, topk, rounding_mode="floor")], bank, local_of[flat[sel]]).to(v.dtype)
    return merge_fn(v.view(rows, topk, x.shape[1]), scores)
