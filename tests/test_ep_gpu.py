"""Expert-parallel mode on 2 GPUs over NCCL: same seeded global batch as the single-GPU operator and the
CPU oracle. Skipped on a box with fewer than 2 GPUs (the CPU-rank version is tests/test_ep_gloo.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mx, combine, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import prime_flash_moe_b200 as P
        from prime_flash_moe_b200 import ep
        T, K, E, N, k = 300, 1024, 16, 1024, 4
        x, w1, w2, ids, wts = O.make_case(T * world, K, E, N, k, seed=11, dist="zipf")
        lo, hi = rank * T, (rank + 1) * T
        if mx:
            (xq, xs), (w1q, w1s), (w2q, w2s) = O.quantize_mx(x), O.quantize_mx(w1), O.quantize_mx(w2)
            experts = ep.LocalExperts(ep.shard_experts(w1q, rank, world).to(dev), ep.shard_experts(w2q, rank, world).to(dev),
                                      P.pack_scales_blocked(ep.shard_experts(w1s, rank, world)).to(dev),
                                      P.pack_scales_blocked(ep.shard_experts(w2s, rank, world)).to(dev))
            layer = ep.ExpertParallelMoE(E, experts, combine=combine)
            assert layer.combine_mode == combine
            # a first step on other routing, then the checked one: the buffers, flags and counts are reused
            layer(xq[lo:hi].to(dev), ids[lo:hi].flip(0).contiguous().to(dev), wts[lo:hi].to(dev), xs[lo:hi].to(dev))
            out = layer(xq[lo:hi].to(dev), ids[lo:hi].to(dev), wts[lo:hi].to(dev), xs[lo:hi].to(dev))
            ref = O.moe_ref_fp32(O.dequantize_mx(xq, xs), O.dequantize_mx(w1q, w1s), O.dequantize_mx(w2q, w2s), ids, wts,
                                 requant_act=True)[lo:hi]
        else:
            experts = ep.LocalExperts(ep.shard_experts(w1, rank, world).to(dev), ep.shard_experts(w2, rank, world).to(dev))
            layer = ep.ExpertParallelMoE(E, experts, combine=combine.split("-")[0])
            assert layer.combine_mode == combine.split("-")[0]
            if combine.startswith("peer"):
                layer.direct_return = combine == "peer-direct"
            layer(x[lo:hi].to(dev), ids[lo:hi].flip(0).contiguous().to(dev), wts[lo:hi].to(dev))
            out = layer(x[lo:hi].to(dev), ids[lo:hi].to(dev), wts[lo:hi].to(dev))
            ref = O.moe_ref_fp32(x, w1, w2, ids, wts)[lo:hi]
        torch.cuda.synchronize()
        from prime_flash_moe_b200 import capi
        assert capi.device_status() == 0
        ret[rank] = (O.max_rel_to_peak(out.cpu(), ref), layer.last_recv_rows, layer.last_sent_rows)
        if layer.exchange is not None:
            layer.exchange.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("combine", ["nccl", "peer", "peer-direct"])
@pytest.mark.parametrize("mx", [False, True])
def test_ep_two_gpus(mx, combine):
    """`nccl`: all-to-all dispatch / combine; `peer`: this library's kernels store rows, slot tables, counts and
    partial sums into the other rank's buffer over NVLink (no NCCL call and no host sync inside a step);
    `peer-direct` (bf16): the down kernel's epilogue adds its results straight into the source rank's buffer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    if mx and combine == "peer-direct":
        pytest.skip("the epilogue-direct return is a bf16 option")
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), mx, combine, ret), nprocs=2, join=True)
    assert len(ret) == 2
    _, _, _, ids, _ = O.make_case(300 * 2, 1024, 16, 1024, 4, seed=11, dist="zipf")
    visits = sum(len(set(int(e) // 8 for e in row)) for row in ids.tolist())      # distinct (token, rank) pairs
    assert sum(ret[r][1] for r in range(2)) == sum(ret[r][2] for r in range(2)) == visits
    for r in range(2):
        assert ret[r][0] <= 2e-2, f"rank {r}: {ret[r][0]}"


@pytest.mark.parametrize("T,E,k,G,dist_name", [(1, 8, 2, 2, "uniform"), (300, 16, 4, 4, "zipf"), (4096, 8, 2, 8, "uniform"),
                                               (5000, 256, 8, 8, "uniform"), (1000, 128, 8, 32, "zipf")])
def test_plan_kernels_match_torch_construction(T, E, k, G, dist_name):
    """pmoe_ep_plan (three kernels, no host sync) against the torch construction of the same plan: bit-exact."""
    from prime_flash_moe_b200 import ep
    ids, wts = O.make_routing(T, E, k, seed=T, dist=dist_name)
    if T >= 300:
        ids[7, 0] = -1          # ids outside [0, E) are ignored
        ids[9, 1] = E
    ref = ep.make_dispatch_plan_torch(ids, wts, E, G)
    got = ep.make_dispatch_plan(ids.cuda(), wts.cuda(), E, G)
    torch.cuda.synchronize()
    V = int(ref.counts.sum())
    assert torch.equal(got.counts.cpu(), ref.counts)
    assert torch.equal(got.visit_token[:V].cpu(), ref.visit_token)
    assert torch.equal(got.visit_meta[:V].cpu(), ref.visit_meta)
    assert torch.equal(got.slot_of.cpu(), ref.slot_of)


def test_single_rank_layer_equals_the_operator():
    """World size 1 (no process group): plan -> LocalExperts -> combine must reproduce the plain operator."""
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import ep
    T, K, E, N, k = 200, 512, 8, 512, 4
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=3)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    dev = "cuda:0"
    layer = ep.ExpertParallelMoE(E, ep.LocalExperts(w1.to(dev), w2.to(dev)))
    out = layer(x.to(dev), ids.to(dev), wts.to(dev))
    torch.cuda.synchronize()
    assert layer.last_sent_rows == T                       # one visit per token on a single rank
    assert O.max_rel_to_peak(out.cpu(), ref) <= 2e-2


def _train_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from prime_flash_moe_b200 import capi, ep
        T, K, E, N, k = 300, 512, 16, 512, 4
        x, w1, w2, ids, wts = O.make_case(T * world, K, E, N, k, seed=17, dist="zipf")
        d_out = torch.randn(T * world, K, generator=torch.Generator().manual_seed(18)).to(torch.bfloat16)
        lo, hi = rank * T, (rank + 1) * T
        per = E // world
        experts = ep.LocalExperts(ep.shard_experts(w1, rank, world).to(dev).requires_grad_(True),
                                  ep.shard_experts(w2, rank, world).to(dev).requires_grad_(True))
        layer = ep.ExpertParallelMoE(E, experts, combine="nccl")
        xr = x[lo:hi].to(dev).requires_grad_(True)
        wr = wts[lo:hi].to(dev).requires_grad_(True)
        out = layer.forward_train(xr, ids[lo:hi].to(dev), wr)
        out.backward(d_out[lo:hi].to(dev))
        torch.cuda.synchronize()
        assert capi.device_status() == 0
        ref = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
        ret[rank] = (O.max_rel_to_peak(out.detach().cpu(), O.moe_ref_fp32(x, w1, w2, ids, wts)[lo:hi]),
                     O.max_rel_to_peak(xr.grad.cpu(), ref[0][lo:hi]),
                     O.max_rel_to_peak(experts.w1.grad.cpu(), ref[1][rank * per:(rank + 1) * per]),
                     O.max_rel_to_peak(experts.w2.grad.cpu(), ref[2][rank * per:(rank + 1) * per]),
                     O.max_rel_to_peak(wr.grad.cpu(), ref[3][lo:hi]))
    finally:
        dist.destroy_process_group()


def test_ep_training_step_two_gpus():
    """forward_train + backward on 2 GPUs over NCCL (kept pre-activations, the library's backward kernels on each
    rank's experts): every rank's d_x / d_topk_weights slice and its experts' weight gradients against autograd
    through the single-process fp32 oracle on the global batch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ret = mp.Manager().dict()
    mp.spawn(_train_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert len(ret) == 2
    for r in range(2):
        for name, err in zip(("out", "d_x", "d_w1", "d_w2", "d_topk_weights"), ret[r]):
            assert err <= 2e-2, f"rank {r} {name}: {err}"


def test_single_rank_training_step():
    """World size 1: forward_train + backward reproduce the gradients of the plain operator's backward pass."""
    from prime_flash_moe_b200 import ep
    T, K, E, N, k = 200, 512, 8, 512, 4
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=5)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    dev = "cuda:0"
    experts = ep.LocalExperts(w1.to(dev).requires_grad_(True), w2.to(dev).requires_grad_(True))
    layer = ep.ExpertParallelMoE(E, experts)
    xr, wr = x.to(dev).requires_grad_(True), wts.to(dev).requires_grad_(True)
    out = layer.forward_train(xr, ids.to(dev), wr)
    out.backward(d_out.to(dev))
    torch.cuda.synchronize()
    ref = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    for got, want in zip((xr.grad, experts.w1.grad, experts.w2.grad, wr.grad), ref):
        assert O.max_rel_to_peak(got.cpu(), want) <= 2e-2
