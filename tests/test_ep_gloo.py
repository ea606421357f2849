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
