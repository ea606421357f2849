"""Expert-parallel mode: the experts of one MoE layer sharded over the ranks of a process group.

Not in the reference (single GPU, single process). One process per GPU; rank ``r`` of ``G`` holds the
contiguous experts ``[r*E/G, (r+1)*E/G)`` (weights and packed scales resident), tokens are data-parallel.
The unit of exchange is a VISIT: a (token, destination rank) pair such that at least one of the token's
``top_k`` experts lives on that rank - a token row crosses NVLink once per visited rank, not once per route
(``top_k=8`` over 8 ranks: 5.25 visits per token on average instead of 8 rows). One step:

1. **plan** (``pmoe_ep_plan`` on the GPU): visits ordered by destination rank, per visit the token, ``top_k``
   slots of (local expert id or -1, routing weight or 0), per rank the visit count; the counts are
   exchanged (all-to-all of ``G`` integers) - the one host sync of the step, NCCL needs split sizes;
2. **dispatch**: one all-to-all of the visiting rows of ``x`` (bf16 rows of ``2K`` bytes, or e4m3 rows of ``K``
   bytes plus ``K/32`` scale bytes) and one of their slot tables - NCCL over NVLink, rows land in the
   receiver's own HBM before any kernel reads them (no remote loads, no TMA multicast anywhere);
3. local compute: ``moe_align`` on the received slot tables (ids of -1 are ignored) and the fused MoE FFN
   kernels of this package on the ``E/G`` local experts with the received routing weights, so the result
   is ONE row per visit: the weighted partial sum over this rank's experts;
4. **combine**: the reverse all-to-all of the bf16 partial sums, then each token's visits are added in fp32 at
   the source rank (``pmoe_ep_combine``).

With ``combine="peer"`` (``"auto"`` picks it when every rank can map its peers' memory) steps 1-4 run without NCCL and
without any host synchronisation: every rank owns one buffer that its peers map through CUDA IPC at set-up
(``PeerExchange``), and the kernels of ``csrc/moe_ep.cu`` store the visiting rows, their slot tables and, on the way
back, the partial sums straight into the destination rank's buffer over NVLink, with per-phase step flags in the
buffer's header (release / acquire, every wait bounded). The visit counts travel the same way (a ``G x G`` matrix in
every header), so each rank computes where its rows land and no split sizes are needed on the host.

The plan has a plain, device-agnostic torch version used for CPU tensors (ranks over ``gloo`` in the tests)
and as the checker of the CUDA one; the expert compute is a callable, by default the CUDA kernels
(``LocalExperts``), which raises without a GPU - there is no CPU implementation of the kernels in this package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Visits of this rank's tokens, ordered by destination rank, tokens ascending inside a rank. Only the first
    ``sum(counts)`` entries of ``visit_token`` / ``visit_meta`` are meaningful."""
    counts: torch.Tensor        # int32 [G]: visits per destination rank
    visit_token: torch.Tensor   # int32 [>= V]: token of each visit
    visit_meta: torch.Tensor    # int32 [>= V, 2*top_k]: local expert ids (-1 = elsewhere) | fp32 weight bits
    slot_of: torch.Tensor       # int32 [T, G]: visit index of (token, rank) or -1


def make_dispatch_plan_torch(topk_ids: torch.Tensor, topk_weights: torch.Tensor, num_experts: int,
                             world_size: int) -> DispatchPlan:
    """Reference construction of the plan with torch ops (any device; synchronises on ``nonzero``)."""
    assert num_experts % world_size == 0, "experts must divide evenly over the ranks"
    per_rank = num_experts // world_size
    T, top_k = topk_ids.shape
    ids = topk_ids.to(torch.int64)
    valid = (ids >= 0) & (ids < num_experts)
    dest = torch.where(valid, torch.div(ids, per_rank, rounding_mode="floor"), torch.zeros_like(ids))
    flags = torch.zeros(T, world_size, dtype=torch.int32, device=ids.device)
    flags.scatter_add_(1, dest, valid.to(torch.int32))
    flags = flags > 0
    gt = torch.nonzero(flags.t().contiguous().view(-1)).view(-1)           # rank-major, tokens ascending
    g, t = torch.div(gt, max(T, 1), rounding_mode="floor"), gt % max(T, 1)
    here = valid[t] & (dest[t] == g.view(-1, 1))                           # [V, top_k]
    local = torch.where(here, ids[t] - g.view(-1, 1) * per_rank, torch.full_like(ids[t], -1)).to(torch.int32)
    w = torch.where(here, topk_weights.view(T, top_k).float()[t], torch.zeros((), device=ids.device))
    meta = torch.cat([local, w.contiguous().view(torch.int32)], dim=1).contiguous()
    slot_of = torch.full((T, world_size), -1, dtype=torch.int32, device=ids.device)
    slot_of[t, g] = torch.arange(gt.numel(), dtype=torch.int32, device=ids.device)
    return DispatchPlan(counts=flags.sum(0).to(torch.int32), visit_token=t.to(torch.int32), visit_meta=meta,
                        slot_of=slot_of)


def make_dispatch_plan(topk_ids: torch.Tensor, topk_weights: torch.Tensor, num_experts: int,
                       world_size: int) -> DispatchPlan:
    """The plan of one step: three small kernels on a GPU (no host sync), torch ops on CPU tensors."""
    assert num_experts % world_size == 0, "experts must divide evenly over the ranks"
    if not topk_ids.is_cuda:
        return make_dispatch_plan_torch(topk_ids, topk_weights, num_experts, world_size)
    T, top_k = topk_ids.shape
    counts, visit_token, visit_meta, slot_of = torch.ops.prime_moe.ep_plan(
        topk_ids.to(torch.int32).contiguous(), topk_weights.reshape(T, top_k).float().contiguous(), num_experts,
        world_size)
    return DispatchPlan(counts, visit_token, visit_meta, slot_of)


def _all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    """Uneven all-to-all along dim 0. 8-bit float rows travel as bytes (NCCL has no e4m3/e8m0 type)."""
    view = rows.view(torch.uint8) if rows.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu) else rows
    out = view.new_empty((sum(recv_counts),) + tuple(view.shape[1:]))
    dist.all_to_all_single(out, view.contiguous(), list(recv_counts), list(send_counts), group=group)
    return out.view(rows.dtype) if view is not rows else out


class LocalExperts:
    """The CUDA path for step 3: this rank's experts through ``moe_align`` + ``fused_moe_*``.

    ``rows[R, K]`` are the visiting token rows, ``local_ids[R, top_k]`` their local expert ids (-1 = no route in
    that slot), ``weights[R, top_k]`` the routing weights; returns the weighted partial sums ``[R, K]`` bf16."""

    def __init__(self, w1, w2, w1_scales=None, w2_scales=None, stages: int = 4, split: bool = True, bpc: int = 0):
        self.w1, self.w2, self.w1_scales, self.w2_scales = w1, w2, w1_scales, w2_scales
        self.stages, self.split = stages, split
        self.num_local = w1.shape[0]
        # CTA pairs (bpc=2) for the bf16 split pipeline on wide layers unless told otherwise: narrow layers are
        # faster on the one-CTA kernels (in-kernel row gather, less padding), and so is mxfp8
        self.bpc = bpc if bpc else (2 if (w1_scales is None and split and w1.shape[1] >= 8192) else 1)

    def __call__(self, rows: torch.Tensor, local_ids: torch.Tensor, weights: torch.Tensor,
                 row_scales: Optional[torch.Tensor] = None, live_rows: Optional[torch.Tensor] = None,
                 out_rows: Optional[torch.Tensor] = None):
        """``live_rows`` (device int32[1]): only that many leading rows are in use, the rest of the worst-case sized
        buffers is neither routed nor zeroed. ``out_rows`` (device int64[R], bf16 only): the address of every
        output row - the results are added there (possibly into a peer's memory) and ``None`` is returned."""
        if not rows.is_cuda:
            raise RuntimeError("LocalExperts needs CUDA tensors: this package has no CPU kernels")
        ops = torch.ops.prime_moe
        R, K = rows.shape
        top_k = local_ids.shape[1]
        if out_rows is not None:
            if not hasattr(self, "_dummy_out") or self._dummy_out.device != rows.device:
                self._dummy_out = torch.zeros(K, dtype=torch.bfloat16, device=rows.device)
            out = self._dummy_out                 # never written: every row goes to its address in out_rows
        else:
            out = torch.empty(R, K, dtype=torch.bfloat16, device=rows.device)   # split=True zeroes it itself
        if R == 0:
            return out
        if not self.split and out_rows is None:
            out.zero_()
        s, e, n = ops.moe_align(local_ids.contiguous(), self.num_local, 128, self.bpc)
        w = weights.reshape(-1).contiguous()
        if live_rows is not None or out_rows is not None:
            from . import capi             # the `_ex` entry points of the C ABI carry the two extras
            if self.w1_scales is None:
                capi.fused_moe_bf16(rows, self.w1, self.w2, s, e, n, w, out, top_k, 128, 64, 4, self.stages, self.bpc, 1,
                                    self.split, live_rows=live_rows, out_rows=out_rows)
            else:
                assert out_rows is None, "direct output rows are a bf16 option"
                capi.fused_moe_mxfp8(rows, row_scales, self.w1, self.w1_scales, self.w2, self.w2_scales, s, e, n, w, out,
                                     top_k, 128, 64, 4, self.stages, self.bpc, self.split, live_rows=live_rows)
        elif self.w1_scales is None:
            ops.fused_moe_bf16(rows, self.w1, self.w2, s, e, n, w, out, top_k, 128, 64, 4, self.stages, self.bpc, 1,
                               self.split)
        else:
            ops.fused_moe_mxfp8(rows, row_scales, self.w1, self.w1_scales, self.w2, self.w2_scales, s, e, n, w, out,
                                top_k, 128, 64, 4, self.stages, self.bpc, self.split)
        return None if out_rows is not None else out


    # ---- training: forward that keeps what the backward pass needs, and the backward pass (bf16 experts only) ----
    def parameters(self):
        return (self.w1, self.w2)

    def forward_keep(self, rows: torch.Tensor, local_ids: torch.Tensor, weights: torch.Tensor):
        """``(y, saved)``: the weighted partial sums as ``__call__`` returns them and what ``backward`` needs (the
        received rows, their routing tables and the gate/up pre-activations the gate/up kernel stored)."""
        if self.w1_scales is not None:
            raise RuntimeError("the backward pass exists for bf16 experts only")
        ops = torch.ops.prime_moe
        R, K = rows.shape
        top_k = local_ids.shape[1]
        out = torch.empty(R, K, dtype=torch.bfloat16, device=rows.device)
        if R == 0:
            return out, None
        s, e, n = ops.moe_align(local_ids.contiguous(), self.num_local, 128, 1)
        w = weights.reshape(-1).contiguous()
        gate_up = ops.fused_moe_bf16_keep(rows, self.w1, self.w2, s, e, n, w, out, top_k)
        return out, (rows, s, e, n, w, gate_up, top_k)

    def backward(self, saved, d_y: torch.Tensor):
        """``(d_rows [R, K] bf16, d_weights [R, top_k] fp32, (d_w1, d_w2))`` for the gradient ``d_y`` of ``y``."""
        if saved is None:
            top_k = 1
            return (d_y.new_empty(0, d_y.shape[1]), torch.empty(0, top_k, dtype=torch.float32, device=d_y.device),
                    (torch.zeros_like(self.w1), torch.zeros_like(self.w2)))
        rows, s, e, n, w, gate_up, top_k = saved
        d_rows, d_w1, d_w2, d_wt = torch.ops.prime_moe.fused_moe_bf16_backward(
            rows, self.w1, self.w2, d_y.contiguous(), s, e, n, w, top_k, gate_up)
        return d_rows, d_wt, (d_w1, d_w2)


class _DeviceBytes:
    """``nbytes`` of device memory at ``ptr`` for ``torch.as_tensor`` (zero-copy view through the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerExchange:
    """The symmetric buffers of the peer-memory exchange: one ``cudaMalloc`` per rank (``pmoe_ep_buffer_alloc``), mapped
    into every other rank through CUDA IPC; handles travel once over the process group at set-up. Layout per rank:
    header | rows [row_cap, row_bytes] | auxiliary rows [row_cap, aux_bytes] | meta int32 [row_cap, 2*top_k] | return
    bf16 [ret_cap, K], with ``row_cap = G * T`` and ``ret_cap = T * min(top_k, G)`` (``T`` = tokens per rank)."""

    def __init__(self, T: int, K: int, top_k: int, row_bytes: int, aux_bytes: int, group=None, device=None):
        import ctypes as C

        from . import capi
        self.lib = capi.lib()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.T, self.K, self.top_k, self.row_bytes, self.aux_bytes = T, K, top_k, row_bytes, aux_bytes
        self.row_cap, self.ret_cap = self.world * T, T * min(top_k, self.world)
        up = lambda v: (v + 1023) // 1024 * 1024
        self.rows_off = up(self.lib.pmoe_ep_header_bytes())
        self.aux_off = up(self.rows_off + self.row_cap * row_bytes)
        self.meta_off = up(self.aux_off + self.row_cap * aux_bytes)
        self.y_off = up(self.meta_off + self.row_cap * 2 * top_k * 4)
        self.nbytes = up(self.y_off + self.ret_cap * K * 2)
        with torch.cuda.device(self.device):
            ptr, handle = C.c_void_p(), C.create_string_buffer(64)
            capi._check(self.lib.pmoe_ep_buffer_alloc(self.nbytes, C.byref(ptr), handle))
            self.local_ptr = ptr.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.peer_ptrs = []
            for g, h in enumerate(handles):
                if g == self.rank:
                    self.peer_ptrs.append(self.local_ptr)
                    continue
                q = C.c_void_p()
                capi._check(self.lib.pmoe_ep_buffer_open(C.create_string_buffer(h, 64), C.byref(q)))
                self.peer_ptrs.append(q.value)
        self.table = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)
        self.buf = torch.as_tensor(_DeviceBytes(self.local_ptr, self.nbytes), device=self.device)
        self.epoch = 0
        dist.barrier(group=group)        # every rank has mapped every buffer before the first store

    def area(self, off: int, rows: int, row_bytes: int) -> torch.Tensor:
        return self.buf[off:off + rows * row_bytes].view(rows, row_bytes)

    def close(self):
        """Unmaps the peers and frees the local buffer; collective (no rank frees while a peer may still store)."""
        if self.local_ptr is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for g, q in enumerate(self.peer_ptrs):
                if g != self.rank:
                    self.lib.pmoe_ep_buffer_close(q)
            dist.barrier(group=self.group)
            self.buf = None
            self.lib.pmoe_ep_buffer_free(self.local_ptr)
        self.local_ptr = None


def peer_exchange_possible(group=None) -> bool:
    """True when this process group is one process per GPU on one node and every GPU can map every other one."""
    if not (dist.is_initialized() and torch.cuda.is_available()) or dist.get_backend(group) == "gloo":
        return False
    world = dist.get_world_size(group)
    if world < 2 or world > torch.cuda.device_count() or world > 32:
        return False
    me = torch.cuda.current_device()
    ok = all(g == me or torch.cuda.can_device_access_peer(me, g) for g in range(torch.cuda.device_count()))
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


class ExpertParallelMoE:
    """``out = layer(x, topk_ids, topk_weights[, x_scales])`` with GLOBAL expert ids in ``topk_ids``.

    ``experts`` is the callable for step 3 (``LocalExperts`` on a GPU). ``last_recv_rows`` holds the number of
    visits this rank computed in the last call and ``last_sent_rows`` the number it sent (load imbalance under
    skewed routing and the saving over one row per route show up there)."""

    def __init__(self, num_experts: int, experts: Callable, group=None, combine: str = "nccl"):
        self.num_experts = num_experts
        self.experts = experts
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._recv_rows = 0
        self._sent_rows = 0
        assert combine in ("nccl", "peer", "auto")
        if combine == "auto":
            combine = "peer" if (self.world > 1 and peer_exchange_possible(group)) else "nccl"
        self.combine_mode = combine if self.world > 1 else "nccl"
        self.exchange: Optional[PeerExchange] = None
        self.direct_return = None   # peer mode: True / False forces the epilogue-direct return, None = by layer shape
        env = __import__("os").environ.get("PMOE_EP_DIRECT")
        if env is not None:
            self.direct_return = env not in ("0", "")
        self.profile = False        # record CUDA events around the phases of a peer-mode step (phase_ms() reads them)
        self._events = []

    # rows this rank computed / sent in the last call; in peer mode the counts stay on the device until asked for
    @property
    def last_recv_rows(self) -> int:
        return int(self._recv_rows.item()) if torch.is_tensor(self._recv_rows) else self._recv_rows

    @property
    def last_sent_rows(self) -> int:
        return int(self._sent_rows.sum().item()) if torch.is_tensor(self._sent_rows) else self._sent_rows

    def _mark(self, name):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events.append((name, ev))

    def phase_ms(self):
        """Mean milliseconds per phase over the profiled steps (synchronises); clears the record."""
        torch.cuda.synchronize()
        sums, n = {}, {}
        prev = None
        for name, ev in self._events:
            if name != "start" and prev is not None:
                sums[name] = sums.get(name, 0.0) + prev.elapsed_time(ev)
                n[name] = n.get(name, 0) + 1
            prev = ev
        self._events = []
        return {k: sums[k] / n[k] for k in sums}

    def _forward_peer(self, x, topk_ids, topk_weights, x_scales=None):
        self._mark("start")
        from . import capi
        T, K = x.shape
        top_k = topk_ids.shape[1]
        row_bytes = K * x.element_size()
        aux_bytes = 0 if x_scales is None else x_scales.shape[1] * x_scales.element_size()
        ex = self.exchange
        if ex is None or (ex.T, ex.K, ex.top_k, ex.row_bytes, ex.aux_bytes) != (T, K, top_k, row_bytes, aux_bytes):
            if ex is not None:
                ex.close()
            ex = self.exchange = PeerExchange(T, K, top_k, row_bytes, aux_bytes, self.group, x.device)
            self._ids = torch.empty(ex.row_cap, top_k, dtype=torch.int32, device=x.device)
            self._wts = torch.empty(ex.row_cap, top_k, dtype=torch.float32, device=x.device)
            self._num_rows = torch.zeros(1, dtype=torch.int32, device=x.device)
            self._out_rows = torch.zeros(ex.row_cap, dtype=torch.int64, device=x.device)
        lib, G, me = ex.lib, self.world, ex.rank
        # wide bf16 layers return their partial sums from the down kernel's epilogue straight into the source ranks'
        # buffers (a long k-loop per tile keeps the NVLink rate low); narrow ones copy finished rows afterwards
        direct = self.direct_return
        if direct is None:
            direct = isinstance(self.experts, LocalExperts) and self.experts.w1.shape[1] >= 8192
        # the epilogue-direct return exists for the bf16 split pipeline of this package's own kernels only
        direct = bool(direct) and x_scales is None and isinstance(self.experts, LocalExperts) and self.experts.split
        plan = make_dispatch_plan(topk_ids, topk_weights, self.num_experts, G)
        ex.epoch += 1
        e, tab, st = ex.epoch, ex.table.data_ptr(), torch.cuda.current_stream().cuda_stream
        x = x.contiguous()
        aux = None if x_scales is None else x_scales.contiguous()
        mark = self._mark
        with torch.cuda.device(x.device):
            if direct:
                ex.buf[ex.y_off:ex.y_off + ex.ret_cap * K * 2].zero_()     # peers ADD into it during this step
            mark("plan")
            capi._check(lib.pmoe_ep_publish_counts(plan.counts.data_ptr(), tab, me, G, e, st))
            capi._check(lib.pmoe_ep_push_rows(x.data_ptr(), row_bytes, 0 if aux is None else aux.data_ptr(), aux_bytes,
                                              plan.visit_token.data_ptr(), plan.visit_meta.data_ptr(), top_k, T, tab,
                                              ex.rows_off, ex.aux_off, ex.meta_off, ex.row_cap, me, G, e, st))
            mark("dispatch")
            capi._check(lib.pmoe_ep_recv_prepare(ex.local_ptr, ex.meta_off, top_k, ex.row_cap, self._ids.data_ptr(),
                                                 self._wts.data_ptr(), self._num_rows.data_ptr(), me, G, e, st))
            mark("wait+prepare")
            rows = ex.area(ex.rows_off, ex.row_cap, row_bytes).view(x.dtype)
            extras = {"live_rows": self._num_rows} if isinstance(self.experts, LocalExperts) else {}
            if direct:
                capi._check(lib.pmoe_ep_return_table(tab, ex.y_off, K, ex.row_cap, ex.ret_cap, me, G,
                                                     self._out_rows.data_ptr(), st))
                extras["out_rows"] = self._out_rows
            if aux is None:
                y = self.experts(rows, self._ids, self._wts, **extras)
            else:
                y = self.experts(rows, self._ids, self._wts, ex.area(ex.aux_off, ex.row_cap, aux_bytes).view(aux.dtype),
                                 **extras)
            mark("experts")
            capi._check(lib.pmoe_ep_push_back(0 if y is None else y.data_ptr(), K, tab, ex.y_off, ex.row_cap, ex.ret_cap,
                                              me, G, e, st))
            mark("return")
            out = torch.empty(T, K, dtype=torch.bfloat16, device=x.device)
            capi._check(lib.pmoe_ep_combine_peer(ex.local_ptr, ex.y_off, plan.slot_of.data_ptr(), out.data_ptr(), T, G, K,
                                                 e, st))
            mark("wait+combine")
        self._recv_rows, self._sent_rows = self._num_rows, plan.counts
        self._keep = (plan, y, x, aux)     # alive until the next call: the kernels above may still be running
        return out

    def forward(self, x, topk_ids, topk_weights, x_scales=None):
        if self.combine_mode == "peer" and x.is_cuda:
            return self._forward_peer(x, topk_ids, topk_weights, x_scales)
        T, K = x.shape
        top_k = topk_ids.shape[1]
        plan = make_dispatch_plan(topk_ids, topk_weights, self.num_experts, self.world)
        if self.world > 1:
            recv_counts = torch.empty_like(plan.counts)
            dist.all_to_all_single(recv_counts, plan.counts, group=self.group)
            send, recv = plan.counts.tolist(), recv_counts.tolist()         # the one host sync of the step
        else:
            send = recv = plan.counts.tolist()
        V = sum(send)
        tokens = plan.visit_token[:V]
        send_rows = x[tokens]
        send_scales = x_scales[tokens] if x_scales is not None else None
        meta = plan.visit_meta[:V]
        if self.world > 1:
            rows = _all_to_all_rows(send_rows, send, recv, self.group)
            meta = _all_to_all_rows(meta, send, recv, self.group)
            scales = _all_to_all_rows(send_scales, send, recv, self.group) if x_scales is not None else None
        else:
            rows, scales = send_rows, send_scales
        self._sent_rows, self._recv_rows = V, rows.shape[0]
        local_ids = meta[:, :top_k].contiguous()
        weights = meta[:, top_k:].contiguous().view(torch.float32)
        y = (self.experts(rows, local_ids, weights, scales) if scales is not None
             else self.experts(rows, local_ids, weights))
        if self.world > 1:
            y = _all_to_all_rows(y, recv, send, self.group)
        return _combine_visits(y, plan.slot_of)

    __call__ = forward

    def forward_train(self, x, topk_ids, topk_weights):
        """The layer as a differentiable function (bf16 experts, NCCL exchange): gradients flow to ``x``,
        ``topk_weights`` and the tensors of ``experts.parameters()``. The backward pass sends the output gradients
        of the visits along the forward dispatch, runs ``experts.backward`` on the rank that owns the experts, and
        returns the row gradients along the forward return (no counterpart in the reference)."""
        return _ExpertParallelTrain.apply(self, x, topk_ids, topk_weights, *self.experts.parameters())


def _combine_visits(y: torch.Tensor, slot_of: torch.Tensor) -> torch.Tensor:
    """out[t] = sum of the rows of the token's visits (bf16, fp32 sum)."""
    if y.is_cuda:
        return torch.ops.prime_moe.ep_combine(y.contiguous(), slot_of)
    slot = slot_of.to(torch.int64)                               # CPU ranks (gloo tests of the host logic)
    K = y.shape[1]
    part = torch.cat([y.float(), torch.zeros(1, K)])[torch.where(slot >= 0, slot, torch.full_like(slot, y.shape[0]))]
    return part.sum(1).to(torch.bfloat16)


class _ExpertParallelTrain(torch.autograd.Function):
    """Forward and backward pass of ``ExpertParallelMoE.forward_train`` (NCCL / gloo exchange)."""

    @staticmethod
    def forward(ctx, layer, x, topk_ids, topk_weights, *params):
        top_k = topk_ids.shape[1]
        plan = make_dispatch_plan(topk_ids, topk_weights.detach(), layer.num_experts, layer.world)
        if layer.world > 1:
            recv_counts = torch.empty_like(plan.counts)
            dist.all_to_all_single(recv_counts, plan.counts, group=layer.group)
            send, recv = plan.counts.tolist(), recv_counts.tolist()
        else:
            send = recv = plan.counts.tolist()
        V = sum(send)
        tokens = plan.visit_token[:V].long()
        rows, meta = x.detach()[tokens], plan.visit_meta[:V]
        if layer.world > 1:
            rows = _all_to_all_rows(rows, send, recv, layer.group)
            meta = _all_to_all_rows(meta, send, recv, layer.group)
        layer._sent_rows, layer._recv_rows = V, rows.shape[0]
        local_ids = meta[:, :top_k].contiguous()
        weights = meta[:, top_k:].contiguous().view(torch.float32)
        y, saved = layer.experts.forward_keep(rows, local_ids, weights)
        if layer.world > 1:
            y = _all_to_all_rows(y, recv, send, layer.group)
        ctx.layer, ctx.saved, ctx.plan, ctx.send, ctx.recv, ctx.tokens = layer, saved, plan, send, recv, tokens
        ctx.ids, ctx.weights_meta = topk_ids, (topk_weights.shape, topk_weights.dtype)
        return _combine_visits(y, plan.slot_of)

    @staticmethod
    def backward(ctx, d_out):
        layer, plan, send, recv = ctx.layer, ctx.plan, ctx.send, ctx.recv
        top_k = ctx.ids.shape[1]
        d_y = d_out.contiguous()[ctx.tokens]                   # out[t] is the plain sum of its visits' rows
        if layer.world > 1:
            d_y = _all_to_all_rows(d_y, send, recv, layer.group)
        d_rows, d_wt, param_grads = layer.experts.backward(ctx.saved, d_y)
        d_rows = d_rows.to(torch.bfloat16)
        d_wt = d_wt.float().reshape(-1, top_k)
        if layer.world > 1:
            d_rows = _all_to_all_rows(d_rows, recv, send, layer.group)
            d_wt = _all_to_all_rows(d_wt.contiguous(), recv, send, layer.group)
        d_x = _combine_visits(d_rows, plan.slot_of)
        # routing weight (t, j) was used by the visit of token t to the rank that owns expert ids[t, j]
        per = layer.num_experts // layer.world
        ids = ctx.ids.to(torch.int64)
        valid = (ids >= 0) & (ids < layer.num_experts)
        dest = torch.where(valid, torch.div(ids, per, rounding_mode="floor"), torch.zeros_like(ids))
        slot = plan.slot_of.to(torch.int64).gather(1, dest)
        ok = valid & (slot >= 0)
        col = torch.arange(top_k, device=ids.device).expand_as(slot)
        if d_wt.shape[0] == 0:
            d_weights = torch.zeros(ids.shape, dtype=torch.float32, device=ids.device)
        else:
            d_weights = torch.where(ok, d_wt[slot.clamp_min(0), col], torch.zeros((), device=ids.device))
        shape, dtype = ctx.weights_meta
        return (None, d_x.to(d_out.dtype), None, d_weights.reshape(shape).to(dtype)) + tuple(param_grads)


def shard_experts(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """This rank's contiguous block of a tensor whose leading dimension is the expert index."""
    per = t.shape[0] // world_size
    return t[rank * per:(rank + 1) * per].contiguous()
