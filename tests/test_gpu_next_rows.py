"""The un-rotated trunk and the banked routed entry against the oracle.

Un-rotated trunk (root.trunkUnrot, src/root.zig:392-420): the device W_std against format.reconstructPublic
(src/core/format.zig:295-331) under the reference's element bar (dense.unrotElemOk, src/core/dense.zig:1953-1963: within one
step of the output dtype at the reference value, or within half a step plus 16 f32 epsilons of the element's absolute term
sum), and y = x W_std against format.project under the dense bars.

Banked entry (deepseek_v41.moeClampedBanked, src/models/deepseek_v41/api.zig:173-200): each row's bytes are moeClamped's on
its bank at top-1 with score 1 (ref.moeRowClamped, src/core/ref.zig:124-190), a skipped id gives a zero row."""
import numpy as np
import pytest
import torch

import turboexl3_b200 as t3
from oracle import binding as ob
from turboexl3_b200 import synth

from gpu_util import HALF_ULP_BF16, HALF_ULP_F16, TORCH_DT, dev, host_f32, record
from test_gpu_moe import check_moe, make_bank

pytestmark = pytest.mark.gpu


def step_of(v: np.ndarray, mant_bits: int) -> np.ndarray:
    """The spacing of a float format with `mant_bits` stored mantissa bits around each |v| (normal range)."""
    e = np.floor(np.log2(np.maximum(np.abs(v), 1e-30)))
    return 2.0 ** (e - mant_bits)


@pytest.mark.parametrize("dt,mant", [("f16", 10), ("bf16", 7)])
@pytest.mark.parametrize("in_dim,out_dim,n,cb", [(256, 384, 64, ob.MUL1), (512, 256, 48, ob.MCG)])
def test_unrot_weight_is_reconstruct_public(dt, mant, in_dim, out_dim, n, cb):
    trellis, suh, svh = synth.linear(31, in_dim, out_dim, n, scaled=True)
    dec = t3.Decode(cb)
    w_t = t3.unrot_build(dev(trellis), dev(suh), dev(svh), dec, TORCH_DT[dt])
    assert w_t.shape == (out_dim, in_dim) and w_t.dtype == TORCH_DT[dt]
    got = w_t.float().cpu().numpy().T.astype(np.float64)  # [in, out]
    what = ob.reconstruct_inner(trellis, in_dim, out_dim, n, cb).view(np.float16).astype(np.float64)
    # the f64 reference diag(suh) H W_hat H diag(svh) (dense.refUnrot, src/core/dense.zig:1921-1940)
    h = np.array([[(-1.0) ** bin(i & k).count("1") for k in range(128)] for i in range(128)])
    ref = np.empty_like(what)
    terms = np.empty_like(what)
    s_in, s_out = suh.view(np.float16).astype(np.float64), svh.view(np.float16).astype(np.float64)
    for rb in range(in_dim // 128):
        for cb_ in range(out_dim // 128):
            tile = what[rb * 128:(rb + 1) * 128, cb_ * 128:(cb_ + 1) * 128]
            scale = np.outer(s_in[rb * 128:(rb + 1) * 128], s_out[cb_ * 128:(cb_ + 1) * 128]) / 128.0
            ref[rb * 128:(rb + 1) * 128, cb_ * 128:(cb_ + 1) * 128] = (h @ tile @ h) * scale
            terms[rb * 128:(rb + 1) * 128, cb_ * 128:(cb_ + 1) * 128] = np.abs(tile).sum() * np.abs(scale)
    d = np.abs(got - ref)
    ok = (d <= step_of(ref, mant)) | (d <= 0.5 * step_of(got, mant) + 16.0 * 2.0 ** -23 * terms)
    assert ok.all(), (dt, int((~ok).sum()), float(d.max()))
    # and against the oracle's own f32 reconstructPublic (f16): equal up to a step of the coarser dtype
    pub = ob.reconstruct_public(trellis, suh, svh, in_dim, out_dim, n, cb).view(np.float16).astype(np.float64)
    assert np.all(np.abs(got - pub) <= 1.01 * step_of(pub, min(mant, 10)) + 1e-7)
    record(f"unrot_weight_{dt}_{in_dim}x{out_dim}", {"max_abs": float(d.max()), "size": int(d.size)})


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("rows", [33, 300])
def test_unrot_linear_is_the_same_map(dt, rows):
    in_dim, out_dim, n = 512, 768, 64
    trellis, suh, svh = synth.linear(32, in_dim, out_dim, n, scaled=True)
    x16 = synth.activations(33, rows, in_dim)
    x = torch.from_numpy(x16.astype(np.float32)).to(TORCH_DT[dt]).cuda()
    w_t = t3.unrot_build(dev(trellis), dev(suh), dev(svh), t3.Decode.mul1, TORCH_DT[dt])
    y = t3.linear_unrot(x, w_t)
    assert y.shape == (rows, out_dim) and y.dtype == x.dtype
    got = host_f32(y)
    # the GEMM itself: x W_std in f64 on the device's own weight, one rounding of each output
    exact = host_f32(x).astype(np.float64) @ w_t.float().cpu().numpy().astype(np.float64).T
    half = HALF_ULP_BF16 if dt == "bf16" else HALF_ULP_F16
    c = ob.compare(got, exact.astype(np.float32), half)["max_ratio"]
    assert c <= 1e-4, c
    # the linear map: format.project's outputs (other roundings: the weight is rounded to dt once, the chain's f16 roundings
    # of xp, z and y are gone)
    want = ob.reconstruct_inner(trellis, in_dim, out_dim, n, ob.MUL1)
    ref = ob.linear_rows_what(host_f32(x), want, suh, svh, in_dim, out_dim)
    r = ob.compare(got, ref)["max_ratio"]
    record(f"unrot_linear_{dt}_rows{rows}", {"compare": r, "gemm_rounded": c, "size": int(got.size)})
    assert r <= (2.5e-2 if dt == "bf16" else 5e-3), r
    with pytest.raises(t3.Exl3Error, match="Exl3EngineNotImplemented"):
        t3.linear_unrot(x[:32].contiguous(), w_t)


def three_banks(seed, hidden, inter, n, counts):
    return [make_bank(seed + i, c, hidden, inter, n) for i, c in enumerate(counts)]


@pytest.mark.parametrize("rows", [1, 7, 32, 64])
@pytest.mark.parametrize("out_dt", ["f32", "bf16"])
def test_banked_rows_are_moe_clamped_on_their_bank(rows, out_dt):
    H, I, n, limit = 512, 256, 48, 7
    banks = three_banks(40, H, I, n, (6, 3, 2))
    rng = np.random.default_rng(41 + rows)
    bank_of = rng.integers(0, 3, rows)
    slot_of = np.array([rng.integers(0, banks[b][1].experts) for b in bank_of])
    ids = (bank_of.astype(np.uint32) << 24) | slot_of.astype(np.uint32)
    if rows >= 7:
        ids[3] = t3.BANKED_SKIP_ID
        ids[5] = ids[1]  # two row-slots on one slot share its decode
    if rows == 64:
        ids[8:50] = ids[0]  # more row-slots on one id than a pass serves
    x16 = synth.activations(42, rows, H)
    x = dev(x16)
    y = t3.moe_clamped_banked(x, [b[0] for b in banks], dev(ids.view(np.int32)), t3.Decode.mul1, limit, TORCH_DT[out_dt])
    assert y.shape == (rows, H) and y.dtype == TORCH_DT[out_dt]
    got = host_f32(y)
    ref = np.zeros((rows, H), np.float32)
    one = np.ones((1, 1), np.float32)
    for r in range(rows):
        if ids[r] == t3.BANKED_SKIP_ID:
            continue
        b, s = int(ids[r] >> 24), int(ids[r] & 0xFFFFFF)
        ref[r] = ob.moe_rows(banks[b][1], x16[r:r + 1].astype(np.float32), np.array([[s]], np.int32), one, ob.MUL1, 16,
                             float(limit), 0)[0]
    skipped = ids == t3.BANKED_SKIP_ID
    assert not got[skipped].any()
    check_moe(got[~skipped], ref[~skipped], out_dt if out_dt == "bf16" else "f16", f"banked_rows{rows}_{out_dt}")
    # the same bytes as the plain clamped call on the row's bank at top-1 with score 1
    r = 0
    b, s = int(ids[r] >> 24), int(ids[r] & 0xFFFFFF)
    plain = t3.moe_clamped(x[r:r + 1].view(1, 1, H), banks[b][0], dev(np.array([[[s]]], np.int32)),
                           dev(np.ones((1, 1, 1), np.float32)), t3.Decode.mul1, limit)
    assert torch.equal(plain.view(-1).to(TORCH_DT[out_dt]).float(), y[r].float())
    assert t3.device_error() == 0


def test_banked_refusals():
    H, I, n = 256, 128, 32
    banks = [b[0] for b in three_banks(50, H, I, n, (2, 2, 2))]
    x = dev(synth.activations(51, 2, H))
    ids = dev(np.array([0, 1], np.int32))
    with pytest.raises(t3.Exl3Error, match="InvalidExl3Clamp"):
        t3.moe_clamped_banked(x, banks, ids, limit=0)
    with pytest.raises(t3.Exl3Error, match="InvalidExl3Clamp"):
        t3.moe_clamped_banked(x, banks, ids, limit=129)
    big = dev(synth.activations(52, 65, H))
    with pytest.raises(t3.Exl3Error, match="BadExl3Shape"):
        t3.moe_clamped_banked(big, banks, dev(np.zeros(65, np.int32)))
    other = make_bank(53, 2, H, 256, n)[0]
    with pytest.raises(t3.Exl3Error, match="BadExl3Shape"):
        t3.moe_clamped_banked(x, [banks[0], other, banks[2]], ids)


@pytest.mark.parametrize("rows,experts,topk", [(1200, 4, 2), (900, 3, 1), (2000, 16, 4)])
def test_routed_prefill_tiles_of_every_height(rows, experts, topk):
    """Experts with more rows than one 128-row tile holds take 256- and 512-row tiles (one decode of the expert's weights
    a tile): a skewed routing puts 1..1000+ rows on an expert, so every height and every remainder rule is met, and each
    row's bytes stay those of the oracle's ref.moeRow."""
    H, I, n = 256, 128, 32
    bank, obank = make_bank(60 + experts, experts, H, I, n)
    rng = np.random.default_rng(61 + rows)
    # skewed: expert 0 takes about half of all slots
    p = np.array([0.5] + [0.5 / (experts - 1)] * (experts - 1))
    inds = np.stack([rng.choice(experts, size=topk, replace=False, p=p) for _ in range(rows)]).astype(np.int32)
    scores = rng.random((rows, topk), dtype=np.float32)
    scores /= scores.sum(1, keepdims=True)
    x16 = synth.activations(62, rows, H)
    y = t3.moe(dev(x16).view(1, rows, H), bank, dev(inds).view(1, rows, topk), dev(scores).view(1, rows, topk))
    counts = np.bincount(inds.reshape(-1), minlength=experts)
    assert counts.max() > 384 and counts.min() >= 1, counts
    ref = ob.moe_rows(obank, x16.astype(np.float32), inds, scores)
    # a maximum over 10^5..10^6 outputs that sum several f16-rounded terms: 1.5 x the bars, as for the full-size layer
    # outputs (achieved at 1200 rows, 4 experts, top-2: compare 6.5e-3, rounded 5.0e-3)
    check_moe(host_f32(y).reshape(rows, H), ref, "f16", f"tile_heights_rows{rows}_e{experts}_k{topk}", terms=1.5)
    assert t3.device_error() == 0


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("rows,topk,experts", [(777, 6, 64), (5, 3, 16), (4096, 10, 512)])
def test_device_dispatch_plan_is_the_host_plan(world, rows, topk, experts):
    """t3_ep_plan (one launch) against parallel.plan_dispatch (torch ops on the host): the same grouping by owning rank,
    the same order inside a rank, each token row once a rank."""
    from turboexl3_b200 import parallel as par
    rng = np.random.default_rng(70 + world + rows)
    inds = np.stack([rng.choice(experts, size=topk, replace=False) for _ in range(rows)]).astype(np.int32)
    order, where, send_rows, meta, counts = t3.ep_plan(dev(inds), experts, world)
    plan = par.plan_dispatch(torch.from_numpy(inds), experts, world)
    c = counts.cpu().tolist()
    assert c[0] == plan.send_counts and c[1] == plan.row_counts
    S = rows * topk
    assert torch.equal(order.cpu().long(), plan.order)
    assert torch.equal(where.cpu().long()[plan.order], torch.arange(S))
    assert torch.equal(send_rows.cpu().long()[:sum(c[1])], plan.send_rows)
    assert torch.equal(meta.cpu()[:, 0], plan.row_in_group) and torch.equal(meta.cpu()[:, 1], plan.local_expert)


def test_mapped_merge_is_the_merge():
    rows, topk, H = 37, 5, 384
    rng = np.random.default_rng(80)
    v = torch.from_numpy(rng.standard_normal((rows * topk, H)).astype(np.float16)).cuda()
    scores = torch.from_numpy(rng.random((rows, topk), dtype=np.float32)).cuda()
    perm = torch.from_numpy(rng.permutation(rows * topk).astype(np.int32)).cuda()  # slot s lies at row perm[s]
    moved = torch.empty_like(v)
    moved[perm.long()] = v
    y0 = t3.moe_merge(v.view(rows, topk, H), scores, torch.float16)
    y1 = t3.moe_merge(moved, scores, torch.float16, where=perm)
    assert torch.equal(y0, y1)


def test_the_launch_plan_names_the_kernels_that_run():
    """t3_plan_linear / t3_plan_moe against the launches themselves: the planned symbol is the kernel the call launched."""
    for rows, n, cb in ((1, 64, t3.MUL1), (12, 48, t3.MCG), (30, 36, t3.MUL1)):
        trellis, suh, svh = synth.linear(90, 512, 384, n, scaled=True)
        t3.linear(dev(synth.activations(91, rows, 512)), dev(trellis), dev(suh), dev(svh), t3.Decode(cb))
        plan = t3.plan_linear(rows, 512, 384, n, t3.Decode(cb))
        assert len(plan) == (1 if rows <= 8 else 2)
        assert t3.last_kernel_symbol() == plan[-1]["symbol"], (rows, n, plan)
    H, I, E, n = 256, 128, 8, 32
    bank, _ = make_bank(92, E, H, I, n)
    for rows, topk in ((3, 2), (5, 1)):
        inds, scores = synth.routing(93, rows, E, topk)
        x = dev(synth.activations(94, rows, H)).view(1, rows, H)
        t3.moe(x, bank, dev(inds).view(1, rows, topk), dev(scores).view(1, rows, topk))
        plan = t3.plan_moe(rows, topk, E, H, I, n)
        assert t3.last_kernel_symbol() == plan[-1]["symbol"], plan
    assert t3.device_error() == 0
