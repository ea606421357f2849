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


def _worker(rank, world, port, mx, ret):
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
            layer = ep.ExpertParallelMoE(E, experts)
            out = layer(xq[lo:hi].to(dev), ids[lo:hi].to(dev), wts[lo:hi].to(dev), xs[lo:hi].to(dev))
            ref = O.moe_ref_fp32(O.dequantize_mx(xq, xs), O.dequantize_mx(w1q, w1s), O.dequantize_mx(w2q, w2s), ids, wts,
                                 requant_act=True)[lo:hi]
        else:
            experts = ep.LocalExperts(ep.shard_experts(w1, rank, world).to(dev), ep.shard_experts(w2, rank, world).to(dev))
            layer = ep.ExpertParallelMoE(E, experts)
            out = layer(x[lo:hi].to(dev), ids[lo:hi].to(dev), wts[lo:hi].to(dev))
            ref = O.moe_ref_fp32(x, w1, w2, ids, wts)[lo:hi]
        torch.cuda.synchronize()
        ret[rank] = (O.max_rel_to_peak(out.cpu(), ref), layer.last_recv_rows)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mx", [False, True])
def test_ep_two_gpus(mx):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), mx, ret), nprocs=2, join=True)
    assert len(ret) == 2
    assert sum(ret[r][1] for r in range(2)) == 300 * 2 * 4
    for r in range(2):
        assert ret[r][0] <= 2e-2, f"rank {r}: {ret[r][0]}"
