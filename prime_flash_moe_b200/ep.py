"""Expert-parallel mode: the experts of one MoE layer sharded over the ranks of a process group.

Not in the reference (single GPU, single process). One process per GPU; rank ``r`` of ``G`` holds the
contiguous experts ``[r*E/G, (r+1)*E/G)`` (weights and packed scales resident), tokens are data-parallel.
One step:

1. every (token, route) pair is assigned to the rank owning its expert; pairs are ordered by destination
   rank (stable), the per-destination counts are exchanged (all-to-all of ``G`` integers);
2. **dispatch**: one all-to-all of the routed rows of ``x`` (bf16 rows of ``2K`` bytes, or e4m3 rows of ``K``
   bytes plus ``K/32`` scale bytes) and one of their local expert ids - NCCL over NVLink, rows land in
   the receiver's own HBM before any kernel reads them (no remote loads, no TMA multicast anywhere);
3. local compute: ``moe_align`` on the received local expert ids (one route per received row) and the
   fused MoE FFN kernels of this package on the ``E/G`` local experts, routing weight 1;
4. **combine**: the reverse all-to-all of the bf16 result rows, then each token's ``top_k`` rows are summed
   with its fp32 routing weights at the source rank.

The index arithmetic (steps 1, 2, 4) is plain, device-agnostic torch and runs unchanged on CPU tensors
over ``gloo``; the expert compute is a callable, by default the CUDA kernels (``LocalExperts``), which
raises without a GPU - there is no CPU implementation of the kernels in this package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Where every (token, route) pair goes. ``perm[i]`` is the pair id sent in slot ``i`` (slots ordered by
    destination rank, pairs in ascending id inside a destination); ``send_counts[g]`` pairs go to rank g."""
    perm: torch.Tensor
    tokens: torch.Tensor          # token of each send slot
    local_expert: torch.Tensor    # expert index on the destination rank, int32
    send_counts: torch.Tensor     # int64 [G]


def make_dispatch_plan(topk_ids: torch.Tensor, num_experts: int, world_size: int) -> DispatchPlan:
    assert num_experts % world_size == 0, "experts must divide evenly over the ranks"
    per_rank = num_experts // world_size
    top_k = topk_ids.shape[1]
    flat = topk_ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, per_rank, rounding_mode="floor")
    perm = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world_size)
    return DispatchPlan(perm=perm, tokens=torch.div(perm, top_k, rounding_mode="floor"),
                        local_expert=(flat[perm] - dest[perm] * per_rank).to(torch.int32),
                        send_counts=send_counts)


def _all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    """Uneven all-to-all along dim 0. 8-bit float rows travel as bytes (NCCL has no e4m3/e8m0 type)."""
    view = rows.view(torch.uint8) if rows.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu) else rows
    out = view.new_empty((sum(recv_counts),) + tuple(view.shape[1:]))
    dist.all_to_all_single(out, view.contiguous(), list(recv_counts), list(send_counts), group=group)
    return out.view(rows.dtype) if view is not rows else out


class LocalExperts:
    """The CUDA path for step 3: this rank's experts through ``moe_align`` + ``fused_moe_*``."""

    def __init__(self, w1, w2, w1_scales=None, w2_scales=None, stages: int = 4, split: bool = True, bpc: int = 0):
        self.w1, self.w2, self.w1_scales, self.w2_scales = w1, w2, w1_scales, w2_scales
        self.stages, self.split = stages, split
        self.num_local = w1.shape[0]
        # CTA pairs (bpc=2) for the bf16 split pipeline on wide layers unless told otherwise: narrow layers are
        # faster on the one-CTA kernels (in-kernel row gather, less padding), and so is mxfp8
        self.bpc = bpc if bpc else (2 if (w1_scales is None and split and w1.shape[1] >= 8192) else 1)

    def __call__(self, rows: torch.Tensor, local_expert: torch.Tensor, row_scales: Optional[torch.Tensor] = None):
        if not rows.is_cuda:
            raise RuntimeError("LocalExperts needs CUDA tensors: this package has no CPU kernels")
        ops = torch.ops.prime_moe
        R, K = rows.shape
        out = torch.empty(R, K, dtype=torch.bfloat16, device=rows.device)   # split=True zeroes it itself
        if R == 0:
            return out
        s, e, n = ops.moe_align(local_expert.reshape(R, 1).contiguous(), self.num_local, 128, self.bpc)
        ones = torch.ones(R, dtype=torch.float32, device=rows.device)
        if self.w1_scales is None:
            ops.fused_moe_bf16(rows, self.w1, self.w2, s, e, n, ones, out, 1, 128, 64, 4, self.stages, self.bpc, 1,
                               self.split)
        else:
            ops.fused_moe_mxfp8(rows, row_scales, self.w1, self.w1_scales, self.w2, self.w2_scales, s, e, n, ones, out,
                                1, 128, 64, 4, self.stages, self.bpc, self.split)
        return out


class ExpertParallelMoE:
    """``out = layer(x, topk_ids, topk_weights[, x_scales])`` with GLOBAL expert ids in ``topk_ids``.

    ``experts`` is the callable for step 3 (``LocalExperts`` on a GPU). ``last_recv_rows`` holds the number of
    rows this rank computed in the last call (load imbalance under skewed routing shows up there)."""

    def __init__(self, num_experts: int, experts: Callable, group=None):
        self.num_experts = num_experts
        self.experts = experts
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.last_recv_rows = 0

    def forward(self, x, topk_ids, topk_weights, x_scales=None):
        T, K = x.shape
        top_k = topk_ids.shape[1]
        plan = make_dispatch_plan(topk_ids, self.num_experts, self.world)
        if self.world > 1:
            recv_counts = torch.empty_like(plan.send_counts)
            dist.all_to_all_single(recv_counts, plan.send_counts, group=self.group)
            # everything that does not need the counts is enqueued before the one host sync of the step
            send_rows = x[plan.tokens]
            send_scales = x_scales[plan.tokens] if x_scales is not None else None
            slots = torch.empty_like(plan.perm)
            slots[plan.perm] = torch.arange(plan.perm.numel(), device=plan.perm.device)
            send, recv = plan.send_counts.tolist(), recv_counts.tolist()
            rows = _all_to_all_rows(send_rows, send, recv, self.group)
            local_e = _all_to_all_rows(plan.local_expert, send, recv, self.group)
            scales = _all_to_all_rows(send_scales, send, recv, self.group) if x_scales is not None else None
        else:
            slots = torch.empty_like(plan.perm)
            slots[plan.perm] = torch.arange(plan.perm.numel(), device=plan.perm.device)
            rows, local_e = x[plan.tokens], plan.local_expert
            scales = x_scales[plan.tokens] if x_scales is not None else None
        self.last_recv_rows = rows.shape[0]
        y = self.experts(rows, local_e, scales) if scales is not None else self.experts(rows, local_e)
        if self.world > 1:
            y = _all_to_all_rows(y, recv, send, self.group)
        # combine at the source: pair p sits in row slots[p]; out[t] = sum_j w[t,j] * y[slots[t*k+j]]
        if y.is_cuda:
            return torch.ops.prime_moe.ep_combine(y, slots, topk_weights.reshape(-1).float().contiguous(), top_k)
        y = y[slots].view(T, top_k, K).float()          # CPU ranks (gloo tests of the host logic)
        return (y * topk_weights.view(T, top_k, 1).float()).sum(1).to(torch.bfloat16)

    __call__ = forward


def shard_experts(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """This rank's contiguous block of a tensor whose leading dimension is the expert index."""
    per = t.shape[0] // world_size
    return t[rank * per:(rank + 1) * per].contiguous()
