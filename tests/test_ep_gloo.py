"""Expert-parallel dispatch / combine logic on CPU ranks (gloo, world_size 2 and 4): the index arithmetic,
the uneven all-to-all exchanges and the weighted combine of prime_flash_moe_b200.ep, with the per-rank
expert compute replaced by the CPU oracle. The assembled result must equal the single-process oracle on
the same global batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from prime_flash_moe_b200 import ep
        T, K, E, N, k, dist_name, mx = case
        x, w1, w2, ids, wts = O.make_case(T * world, K, E, N, k, seed=3, dist=dist_name)
        if mx:
            (xq, xs), (w1q, w1s), (w2q, w2s) = O.quantize_mx(x), O.quantize_mx(w1), O.quantize_mx(w2)
            w1d, w2d = O.dequantize_mx(w1q, w1s), O.dequantize_mx(w2q, w2s)
        else:
            w1d, w2d = w1, w2
        lo, hi = rank * T, (rank + 1) * T
        w1_loc, w2_loc = ep.shard_experts(w1d, rank, world), ep.shard_experts(w2d, rank, world)

        n_loc = w1_loc.shape[0]
        # slots that route elsewhere carry id -1 and weight 0: send them to an all-zero extra expert
        w1_ext = torch.cat([w1_loc.float(), torch.zeros(1, N, K)])
        w2_ext = torch.cat([w2_loc.float(), torch.zeros(1, K, N // 2)])

        def experts(rows, local_ids, weights, row_scales=None):
            r = rows if row_scales is None else O.dequantize_mx(rows, row_scales)
            if r.shape[0] == 0:
                return torch.zeros(0, K, dtype=torch.bfloat16)
            assert int(local_ids.max()) < n_loc and bool(((local_ids >= 0) | (weights == 0)).all())
            assert bool((local_ids >= 0).any(1).all()), "a visit without a route on this rank"
            ids = torch.where(local_ids < 0, torch.full_like(local_ids, n_loc), local_ids)
            return O.moe_ref_fp32(r, w1_ext, w2_ext, ids, weights, requant_act=mx).to(torch.bfloat16)

        layer = ep.ExpertParallelMoE(E, experts)
        if mx:
            out = layer(xq[lo:hi], ids[lo:hi], wts[lo:hi], xs[lo:hi])
            ref = O.moe_ref_fp32(O.dequantize_mx(xq, xs), w1d, w2d, ids, wts, requant_act=True)[lo:hi]
        else:
            out = layer(x[lo:hi], ids[lo:hi], wts[lo:hi])
            ref = O.moe_ref_fp32(x, w1d, w2d, ids, wts)[lo:hi]
        # received visits over all ranks = sent visits over all ranks = distinct (token, rank) pairs of the batch
        rows = torch.tensor([layer.last_recv_rows, layer.last_sent_rows])
        dist.all_reduce(rows)
        per = E // world
        visits = sum(len(set((int(e) // per) for e in row)) for row in ids.tolist())
        ret[rank] = (O.max_rel_to_peak(out, ref), int(rows[0]), int(rows[1]), visits)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", [
    (48, 128, 8, 256, 2, "uniform", False),
    (33, 128, 16, 256, 4, "zipf", False),      # skewed: uneven splits
    (5, 128, 4, 256, 1, "uniform", False),     # few tokens: some ranks receive little or nothing
    (40, 256, 8, 256, 2, "uniform", True),     # mxfp8 rows + scale rows dispatched as bytes
])
def test_ep_matches_single_process_oracle(world, case):
    T, K, E, N, k, _, _ = case
    if E % world:
        pytest.skip("experts must divide over ranks")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err, received, sent, visits = ret[rank]
        assert err <= 1e-2, f"rank {rank}: {err}"          # bf16 rounding of the partial sums only
        assert received == sent == visits <= T * world * min(k, world)


def test_dispatch_plan_visits():
    """The torch construction of the plan (the checker of the CUDA one): visits ordered by rank then token, slot
    tables holding exactly the routes of that rank, slot_of the inverse map."""
    from prime_flash_moe_b200 import ep
    T, E, k, G = 64, 16, 4, 4
    ids, wts = O.make_routing(T, E, k, seed=1, dist="zipf")
    plan = ep.make_dispatch_plan(ids, wts, E, G)
    per = E // G
    V = int(plan.counts.sum())
    tok, meta = plan.visit_token[:V].long(), plan.visit_meta[:V]
    local, w = meta[:, :k], meta[:, k:].contiguous().view(torch.float32)
    g_of = torch.repeat_interleave(torch.arange(G), plan.counts.long())
    assert torch.all(g_of[1:] >= g_of[:-1])
    for g in range(G):
        seg = tok[g_of == g]
        assert torch.all(seg[1:] > seg[:-1])                                 # tokens ascending inside a rank
    for v in range(V):
        t, g = int(tok[v]), int(g_of[v])
        for j in range(k):
            e = int(ids[t, j])
            if e // per == g:
                assert int(local[v, j]) == e - g * per and float(w[v, j]) == float(wts[t, j])
            else:
                assert int(local[v, j]) == -1 and float(w[v, j]) == 0.0
        assert int(plan.slot_of[t, g]) == v
    assert int((plan.slot_of >= 0).sum()) == V
    expected = sum(len(set(int(e) // per for e in row)) for row in ids.tolist())
    assert V == expected


class _TorchExperts:
    """Stand-in for ep.LocalExperts on CPU ranks: the fp32 oracle and autograd through it (slots routed elsewhere
    carry id -1 and weight 0 and go to an all-zero extra expert)."""

    def __init__(self, w1_loc, w2_loc):
        self.w1, self.w2 = w1_loc.float(), w2_loc.float()

    def parameters(self):
        return (self.w1, self.w2)

    def forward_keep(self, rows, local_ids, weights):
        n_loc, N, K = self.w1.shape
        leaves = [t.detach().float().clone().requires_grad_(True) for t in (rows, weights, self.w1, self.w2)]
        if rows.shape[0] == 0:
            return torch.zeros(0, K, dtype=torch.bfloat16), None
        ids = torch.where(local_ids < 0, torch.full_like(local_ids, n_loc), local_ids)
        with torch.enable_grad():           # called from inside an autograd.Function, where recording is off
            w1_ext = torch.cat([leaves[2], torch.zeros(1, N, K)])
            w2_ext = torch.cat([leaves[3], torch.zeros(1, K, N // 2)])
            y = O.moe_ref_fp32(leaves[0], w1_ext, w2_ext, ids, leaves[1])
        return y.detach().to(torch.bfloat16), (leaves, y)

    def backward(self, saved, d_y):
        if saved is None:
            return (torch.zeros(0, self.w1.shape[2]), torch.zeros(0, 1), (torch.zeros_like(self.w1), torch.zeros_like(self.w2)))
        leaves, y = saved
        y.backward(d_y.float())
        return leaves[0].grad, leaves[1].grad, (leaves[2].grad, leaves[3].grad)


def _train_worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from prime_flash_moe_b200 import ep
        T, K, E, N, k, dist_name = case
        x, w1, w2, ids, wts = O.make_case(T * world, K, E, N, k, seed=13, dist=dist_name)
        d_out = torch.randn(T * world, K, generator=torch.Generator().manual_seed(14)).to(torch.bfloat16)
        lo, hi = rank * T, (rank + 1) * T
        per = E // world
        experts = _TorchExperts(ep.shard_experts(w1, rank, world), ep.shard_experts(w2, rank, world))
        for p in experts.parameters():
            p.requires_grad_(True)
        layer = ep.ExpertParallelMoE(E, experts)
        xr = x[lo:hi].float().requires_grad_(True)
        wr = wts[lo:hi].clone().requires_grad_(True)
        out = layer.forward_train(xr, ids[lo:hi], wr)
        out.backward(d_out[lo:hi])
        ref = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
        fwd = O.moe_ref_fp32(x, w1, w2, ids, wts)[lo:hi]
        errs = (O.max_rel_to_peak(out, fwd),
                O.max_rel_to_peak(xr.grad, ref[0][lo:hi]),
                O.max_rel_to_peak(experts.w1.grad, ref[1][rank * per:(rank + 1) * per]),
                O.max_rel_to_peak(experts.w2.grad, ref[2][rank * per:(rank + 1) * per]),
                O.max_rel_to_peak(wr.grad, ref[3][lo:hi]))
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", [
    (24, 64, 8, 128, 2, "uniform"),
    (17, 64, 16, 128, 4, "zipf"),
    (3, 64, 4, 128, 1, "uniform"),      # few tokens: some ranks receive nothing
])
def test_ep_training_step_matches_autograd_oracle(world, case):
    """forward_train + backward over CPU ranks: the gradient exchanges (output gradients along the dispatch, row and
    routing-weight gradients along the return) and the slot arithmetic, with the per-rank expert compute replaced
    by autograd through the fp32 oracle. Every rank's d_x / d_topk_weights slice and its experts' weight gradients
    must equal autograd through the single-process oracle on the global batch."""
    if case[2] % world:
        pytest.skip("experts must divide over ranks")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_train_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        for name, err in zip(("out", "d_x", "d_w1", "d_w2", "d_topk_weights"), ret[rank]):
            assert err <= 1e-2, f"rank {rank} {name}: {err}"
