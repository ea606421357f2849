#!/usr/bin/env python
"""Benchmark of the fused MoE FFN hot path (moe_align -> gate/up GEMM -> SwiGLU -> down GEMM -> top-k reduce).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1] [--dtype bf16] [--impl ours|reference|cpu]

Prints ONE JSON line (rank 0). A step = one pass of the hot path over one synthetic batch:
`torch.ops.prime_moe.moe_align` + `torch.ops.prime_moe.fused_moe_*`. `value` is whole-job TFLOP/s with
the inputs resident in HBM (algorithmic FLOPs 3*P*K*N, P = T*top_k; padding rows do not count);
`e2e` is the same metric with the step's activations, routing ids and routing weights copied from pinned
host memory and `out` copied back inside the timed region (weights stay resident, as in a model); the copies
of neighbouring steps run on their own streams beside the kernels (two sets of device buffers), as a caller
feeding the layer from host memory would do. Both arms use the same harness.

`--impl reference` times the UNMODIFIED reference (pip-installed into baseline/_ref from the reference
checkout) through its own public API on the same workload, its best accepted knob setting chosen during
warm-up. The reference has no CPU implementation of this path - its product is sm_100a kernels - so that
arm runs on the GPU too; the reference's only CPU code for the path, the PyTorch MoE of its tests, is
timed as `cpu_baseline` (and alone with `--impl cpu`).

After the headline workload the default single-GPU run measures a short fixed SWEEP of the other benchmark
configurations (c0; c2 at T = 16, 128, 8192 in bf16 and mxfp8; c3 mxfp8; c4 bf16 and mxfp8; `moe_align` alone at the
c4 and c3 sizes) and attaches it as `sweep`: per entry the step time, TFLOP/s and the roofline of its dominant
kernel (tensor-bound entries against the measured tensor peak, weight-streaming ones and `moe_align` against the
measured HBM copy bandwidth). `--impl reference` measures the same entries with the reference's kernels, so every
entry has the reference's time beside it. `--no-sweep` skips it.

N > 1 (torchrun): expert-parallel mode when the experts divide over the ranks (`--parallel ep`, the default
then: NCCL all-to-all dispatch / combine), else every rank runs its own batch against a full replica of the
experts (`--parallel replica`, no collective on the data path). Weak scaling either way.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

CONFIGS = {
    # name: (T, K, E, N, top_k, routing)
    "c0": (256, 4096, 8, 512, 4, "uniform"),
    "c1": (4096, 4096, 8, 28672, 2, "uniform"),            # Mixtral-8x7B layer: the headline workload
    "c2": (8192, 2048, 128, 1536, 8, "uniform"),           # Qwen3-30B-A3B layer (T overridable with --tokens)
    "c3": (16384, 7168, 256, 4096, 8, "uniform"),          # DeepSeek-V3 layer
    "c4": (65536, 4096, 128, 3072, 8, "zipf"),             # skewed routing stress
    "refbench": (16384, 2048, 32, 2048, 4, "uniform"),     # the reference benchmark's default shape
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "cpu"])
    ap.add_argument("--config", default="c1", choices=sorted(CONFIGS))
    ap.add_argument("--tokens", type=int, default=0, help="override T of the configuration")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "mxfp8"])
    ap.add_argument("--split", type=int, default=1)
    ap.add_argument("--stages", type=int, default=4)
    ap.add_argument("--warp-n", type=int, default=4, choices=[4, 8],
                    help="epilogue warps of the bf16 kernels: (block_n, warp_n) = (64, 4) or (32, 8)")
    ap.add_argument("--bpc", type=int, default=0, help="0 = 2 (CTA pairs) for bf16 split, 1 otherwise")
    ap.add_argument("--parallel", default="auto", choices=["auto", "replica", "ep"],
                    help="N > 1: 'ep' shards the experts over the ranks (NCCL all-to-all dispatch/combine, the "
                         "default when the expert count divides), 'replica' runs N independent copies")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="headline workload only")
    ap.add_argument("--op", default="moe", choices=["moe", "moe_align", "pre", "backward", "train"],
                    help="'moe_align' times the routing kernels alone on the routing table of --config (GB/s line); "
                         "'pre' times the router and the MX activation quantiser alone at the c3 shapes; 'backward' times the "
                         "bf16 backward pass and each of its steps on --config; 'train' times forward + backward of the bf16 "
                         "layer (expert-parallel under torchrun)")
    ap.add_argument("--ep-combine", default="auto", choices=["auto", "nccl", "peer"],
                    help="expert-parallel combine: NCCL all-to-all, or this library's kernel storing into the source "
                         "rank's buffer over NVLink (auto = peer when every rank can map its peers)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def dist_setup(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    return world, rank, local


def bind_to_gpu_numa_node(index: int):
    """Multi-rank runs: keep this process (and the pinned host buffers it allocates afterwards) on the CPUs NVML
    reports as local to its GPU, so that eight ranks copying through host memory do not all cross the socket link.
    Reads the affinity mask only; any failure (no NVML, CPUs outside the container's cpuset) leaves things as they are."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def barrier_sync(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int, device) -> float:
    if world == 1:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def make_inputs(cfg, seed, device, weights=True):
    """Seeded synthetic batch: x ~ N(0,1) bf16, w1 ~ N(0,1/K), w2 ~ N(0,1/H) bf16 generated on the device;
    routing (distinct experts per token, uniform or Zipf s=1.2) and softmax weights from the CPU oracle's
    generator so that every arm sees identical routing."""
    import torch
    sys.path.insert(0, str(ROOT))
    from oracle import moe_oracle as O
    T, K, E, N, k, routing = cfg
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(T, K, device=device, generator=g).to(torch.bfloat16)
    w1 = w2 = None
    if weights:
        w1 = torch.randn(E, N, K, device=device, generator=g, dtype=torch.bfloat16) * K ** -0.5
        w2 = torch.randn(E, K, N // 2, device=device, generator=g, dtype=torch.bfloat16) * (N // 2) ** -0.5
    ids, wts = O.make_routing(T, E, k, seed + 1, routing)
    return x, w1, w2, ids, wts


def quantize_mx_device(t, block=32):
    """The OCP-MX quantiser of the reference's tests (test/test_mxfp8.py:21-38) on whatever device `t` is on."""
    import torch
    k = t.shape[-1]
    g = t.float().reshape(*t.shape[:-1], k // block, block)
    bits = g.abs().amax(-1).contiguous().view(torch.int32)
    e = (((bits >> 23) & 0xFF) - 8).clamp(0, 254)
    inv = torch.exp2((127 - e).float())
    q = (g * inv.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(*t.shape[:-1], k).contiguous(), e.to(torch.uint8).view(torch.float8_e8m0fnu)


def quantize_mx_weights(w, chunk=16):
    """`quantize_mx_device` over a weight tensor [E, rows, cols], a few experts at a time (bounded fp32 temporaries)."""
    import torch
    qs, ss = [], []
    for i in range(0, w.shape[0], chunk):
        q, sc = quantize_mx_device(w[i:i + chunk])
        qs.append(q), ss.append(sc)
    return torch.cat(qs), torch.cat(ss)


def pack_scales(scales):
    """Blocked scale layout (prime_moe/__init__.py:106-115); plain torch so that both arms can use it."""
    import torch
    u = scales.view(torch.uint8)
    lead = u.shape[:-2]
    mn, kb = u.shape[-2:]
    t = u.reshape(-1, mn // 128, 4, 32, kb // 4, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
    return t.reshape(*lead, -1).view(torch.float8_e8m0fnu)


def time_cpu_oracle(x, w1, w2, ids, wts, sample_tokens):
    """The reference's PyTorch MoE (restated in oracle/) on the host cores, on the first
    `sample_tokens` tokens of the batch. Returns (TFLOP/s, seconds, threads)."""
    import torch
    from oracle import moe_oracle as O
    T = min(sample_tokens, x.shape[0])
    K = x.shape[1]
    N = w1.shape[1]
    xs, ids_s, wts_s = x[:T].cpu(), ids[:T].cpu(), wts[:T].cpu()
    w1c, w2c = w1.cpu(), w2.cpu()
    O.moe_ref_grouped_mm(xs[:8], w1c, w2c, ids_s[:8], wts_s[:8])   # warm-up (thread pool, allocator)
    t0 = time.perf_counter()
    O.moe_ref_grouped_mm(xs, w1c, w2c, ids_s, wts_s)
    dt = time.perf_counter() - t0
    flops = 3.0 * T * ids.shape[1] * K * N
    return flops / dt / 1e12, dt, torch.get_num_threads()


def roofline_mxfp8(args, capi, ops, tensors, ids, wts, out, cfg, peaks, whole_tflops, flush_buf=None):
    """Gate/up kernel of the mxfp8 split pipeline timed alone (profiling hook). The denominator is a cuBLASLt
    block-scaled mxfp8 GEMM timed in the same run (`measure_mxfp8_peak`)."""
    import torch
    T, K, E, N, k, _ = cfg
    xq, xs, w1q, w1s, w2q, w2s = tensors
    lib = capi.lib()
    s, e, n = ops.moe_align(ids, E, 128, 1)
    nbytes = lib.pmoe_fused_moe_mxfp8_workspace_bytes(T, K, N, s.numel(), 1)
    ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=out.device)
    off = (-ws.data_ptr()) % 1024
    ws = ws[off:off + nbytes]
    call = lambda: capi.fused_moe_mxfp8(xq, xs, w1q, w1s, w2q, w2s, s, e, n, wts, out, k, 128, 64, 4, args.stages, 1, True,
                                        workspace=ws)
    call()
    per_kernel = {}
    for name, mask in (("gather_rows_mxfp8", 1), ("moe_up_mxfp8", 2), ("moe_down_mxfp8", 4)):
        lib.pmoe_debug_set_phase_mask(mask)
        per_kernel[name] = time_calls(call, 20, flush_buf)
    lib.pmoe_debug_set_phase_mask(7)
    call()
    torch.cuda.synchronize()
    achieved = 2.0 * T * k * K * N / (per_kernel["moe_up_mxfp8"] * 1e-3) / 1e12
    peak, source = measure_mxfp8_peak(out.device)
    assert capi.device_status() == 0
    return {"kernel": "moe_up_mxfp8_kernel", "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "peak_source": source,
            "traffic": 0.6565e9 if (args.config == "c2" and not args.tokens) else None,   # from the ncu capture summarised under profiles/
            "kernel_ms": per_kernel, "whole_op_frac": whole_tflops / peak}


def select_knobs(candidates, trial_calls=3, final_calls=8):
    """The reference arm's knob choice: every candidate `(call, knobs)` is timed over `trial_calls` calls after two
    warm-up calls, then the three fastest are timed again over `final_calls` calls and the fastest of those wins
    (a single short trial picked a slow setting now and then). Returns `(ms, call, knobs)` or None."""
    import torch

    def timed(call, n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            call()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    first = []
    for call, knobs in candidates:
        try:
            for _ in range(2):
                call()
            torch.cuda.synchronize()
            first.append((timed(call, trial_calls), call, knobs))
        except Exception:
            continue
    if not first:
        return None
    first.sort(key=lambda t: t[0])
    second = [(timed(call, final_calls), call, knobs) for _, call, knobs in first[:3]]
    return min(second, key=lambda t: t[0])


def time_calls(call, reps, flush_buf=None):
    """Mean milliseconds of `call` on the current stream: one pair of events around `reps` back-to-back calls,
    or - with a flush buffer - a pair per call with the L2 flushed (buffer rewritten) before each."""
    import torch
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    if flush_buf is None:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            call()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps
    pairs = []
    for _ in range(reps):
        flush_buf.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        call()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in pairs) / reps


def weight_streaming_roofline(roof, cfg, ids, per_kernel_up_ms, ms_step, peaks, mx, traffic):
    """Calls with fewer than 256 routed rows per expert are bound by streaming the weights of the experts
    actually routed to, not by the tensor pipe: restate the roofline of the gate/up kernel against the
    measured HBM copy bandwidth. Algorithmic bytes of that kernel: w1 of the touched experts (+ scales),
    the routed rows of x, the activation written, `out` zeroed."""
    T, K, E, N, k, _ = cfg
    if T * k >= 256 * E:
        return roof
    touched = int(ids.unique().numel())
    wbytes = 1.0 + 1.0 / 32 if mx else 2.0
    abytes = 1.0 + 1.0 / 32 if mx else 2.0
    up_bytes = touched * N * K * wbytes + T * k * K * abytes + T * k * (N // 2) * abytes + T * K * 2
    op_bytes = touched * (N * K + K * (N // 2)) * wbytes + T * K * abytes + T * K * 2
    achieved = up_bytes / (per_kernel_up_ms * 1e-3) / 1e9
    roof = dict(roof)
    roof.update({"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                 "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"] + " (STREAM-style copy)",
                 "traffic": traffic, "algorithmic_bytes": up_bytes, "experts_touched": touched,
                 "whole_op_frac": op_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                 })
    roof.pop("frac_of_sustained", None)
    return roof


_MX_PEAK = None


def measure_mxfp8_peak(device):
    global _MX_PEAK
    if _MX_PEAK is None:
        _MX_PEAK = _measure_mxfp8_peak(device)
    return _MX_PEAK


def _measure_mxfp8_peak(device):
    """MEASURED_PEAKS.json has no fp8 figure, so the denominator is measured here the way the bf16 one was:
    cuBLASLt block-scaled (e4m3 x e8m0/32) 8192^3 through torch._scaled_mm, best of 10 (burst).
    2930 TFLOP/s (an earlier B200 measurement of the same GEMM; per-tensor-scaled fp8: 3151) is used if the call is
    unavailable, and the line says so."""
    import torch
    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        sa = torch.full((n, n // 32), 127, dtype=torch.uint8, device=device).view(torch.float8_e8m0fnu)
        sb = torch.full((n, n // 32), 127, dtype=torch.uint8, device=device).view(torch.float8_e8m0fnu)
        fn = lambda: torch._scaled_mm(a, b, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        return 2.0 * n ** 3 / best / 1e9, "measured in this run (cuBLASLt mxfp8 block-scaled 8192^3, burst)"
    except Exception:
        return 2930.0, "earlier B200 measurement (cuBLASLt mxfp8 block-scaled 8192^3, burst); torch._scaled_mm unavailable here"



# ------------------------------------------------------------------------------------------------
# sweep: the other benchmark configurations, short runs, one compact entry each
# ------------------------------------------------------------------------------------------------
SWEEP = [
    # (configuration, T override or 0, dtype)
    ("c0", 0, "bf16"),
    ("c2", 16, "bf16"), ("c2", 16, "mxfp8"), ("c2", 128, "bf16"), ("c2", 128, "mxfp8"),
    ("c2", 8192, "bf16"), ("c2", 8192, "mxfp8"),
    ("c3", 0, "mxfp8"),
    ("c4", 0, "bf16"), ("c4", 0, "mxfp8"),
]
SWEEP_ALIGN = ["c4", "c3"]


def build_sweep_case(name, tokens, dtype, device):
    """Seeded inputs of one sweep entry, generated on the device 16 experts at a time so that the bf16 originals of
    a large mxfp8 layer never exist all at once. Both arms call this, so they see identical tensors."""
    import torch
    sys.path.insert(0, str(ROOT))
    from oracle import moe_oracle as O
    T, K, E, N, k, routing = CONFIGS[name]
    if tokens:
        T = tokens
    seed = 4321 + sorted(CONFIGS).index(name)
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(T, K, device=device, generator=g).to(torch.bfloat16)
    mx = dtype == "mxfp8"
    w1p, w2p, w1sp, w2sp = [], [], [], []
    for e0 in range(0, E, 16):
        n = min(16, E - e0)
        a = torch.randn(n, N, K, device=device, generator=g, dtype=torch.bfloat16) * K ** -0.5
        b = torch.randn(n, K, N // 2, device=device, generator=g, dtype=torch.bfloat16) * (N // 2) ** -0.5
        if mx:
            q, sc = quantize_mx_device(a)
            w1p.append(q), w1sp.append(pack_scales(sc))
            q, sc = quantize_mx_device(b)
            w2p.append(q), w2sp.append(pack_scales(sc))
        else:
            w1p.append(a), w2p.append(b)
    ids, wts = O.make_routing(T, E, k, seed + 1, routing)
    case = {"cfg": (T, K, E, N, k, routing), "ids_cpu": ids, "ids": ids.to(device), "wts": wts.to(device), "x": x,
            "w1": torch.cat(w1p), "w2": torch.cat(w2p)}
    if mx:
        case["w1s"], case["w2s"] = torch.cat(w1sp), torch.cat(w2sp)
        case["xq"], case["xs"] = quantize_mx_device(x)
    return case


def time_steps(step, steps, flush_buf):
    """Mean ms of `step` (3 warm-up calls first): back to back, or with the L2 flushed before every timed call."""
    return time_calls(step, steps, flush_buf)


def sweep_entry_ours(name, tokens, dtype, device, peaks, stages):
    import torch
    from prime_flash_moe_b200 import capi
    ops = torch.ops.prime_moe
    mx = dtype == "mxfp8"
    c = build_sweep_case(name, tokens, dtype, device)
    T, K, E, N, k, routing = c["cfg"]
    bpc = 2 if (not mx and N >= 8192) else 1
    out = torch.empty(T, K, dtype=torch.bfloat16, device=device)
    touched = int(c["ids_cpu"].unique().numel())
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device) if \
        touched * (N * K + K * (N // 2)) * (1 if mx else 2) < (256 << 20) else None

    def step():
        s, e, n = ops.moe_align(c["ids"], E, 128, bpc)
        if mx:
            ops.fused_moe_mxfp8(c["xq"], c["xs"], c["w1"], c["w1s"], c["w2"], c["w2s"], s, e, n, c["wts"], out, k, 128, 64, 4,
                                stages, bpc, True)
        else:
            ops.fused_moe_bf16(c["x"], c["w1"], c["w2"], s, e, n, c["wts"], out, k, 128, 64, 4, stages, bpc, 1, True)

    flops = 3.0 * T * k * K * N
    steps = 20 if flops < 5e12 else 8
    ms = time_steps(step, steps, flush_buf)
    # the gate/up kernel alone (2/3 of the FLOPs, and of the weight bytes) through the profiling hook
    lib = capi.lib()
    s, e, n = ops.moe_align(c["ids"], E, 128, bpc)
    wsb = (lib.pmoe_fused_moe_mxfp8_workspace_bytes if mx else lib.pmoe_fused_moe_bf16_workspace_bytes)(T, K, N, s.numel(), 1)
    ws = torch.empty(wsb + 1024, dtype=torch.uint8, device=device)
    off = (-ws.data_ptr()) % 1024
    ws = ws[off:off + wsb]
    if mx:
        call = lambda: capi.fused_moe_mxfp8(c["xq"], c["xs"], c["w1"], c["w1s"], c["w2"], c["w2s"], s, e, n, c["wts"], out, k,
                                            128, 64, 4, stages, bpc, True, workspace=ws)
    else:
        call = lambda: capi.fused_moe_bf16(c["x"], c["w1"], c["w2"], s, e, n, c["wts"], out, k, 128, 64, 4, stages, bpc, 1,
                                           True, workspace=ws)
    lib.pmoe_debug_set_phase_mask(2)
    up_ms = time_calls(call, 10, flush_buf)
    lib.pmoe_debug_set_phase_mask(4)
    down_ms = time_calls(call, 10, flush_buf)
    lib.pmoe_debug_set_phase_mask(7)
    call()
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a kernel recorded an error status"
    wb = (1.0 + 1.0 / 32) if mx else 2.0
    up_bytes = touched * N * K * wb + T * k * K * wb + T * k * (N // 2) * wb + T * K * 2
    kernel = ("moe_up_mxfp8_kernel" if mx else ("moe_pair_bf16_kernel<up>" if bpc == 2 else "moe_up_bf16_kernel (or its "
              "two-block variant)"))
    if T * k >= 256 * E:       # compute-bound call: tensor roofline of the gate/up kernel
        peak, src = measure_mxfp8_peak(device) if mx else (peaks["bf16_tflops"], peaks["source"] + " (burst cuBLAS bf16)")
        ach = 2.0 * T * k * K * N / (up_ms * 1e-3) / 1e12
        roof = {"kernel": kernel, "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "peak_source": src, "traffic": None, "algorithmic_bytes": up_bytes}
    else:                      # weight streaming: the experts actually routed to, at the measured copy bandwidth
        ach = up_bytes / (up_ms * 1e-3) / 1e9
        roof = {"kernel": kernel, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"] + " (STREAM-style copy)", "traffic": None,
                "algorithmic_bytes": up_bytes, "experts_touched": touched}
    roof["kernel_ms"] = {"up": up_ms, "down": down_ms}
    del c, ws, out, flush_buf
    torch.cuda.empty_cache()
    return {"config": name, "tokens": T, "dtype": dtype, "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "tokens_per_s": T / (ms * 1e-3), "l2_flushed": touched * (N * K + K * (N // 2)) * (1 if mx else 2) < (256 << 20),
            "roofline": roof}


def sweep_entry_reference(name, tokens, dtype, device, ref_pkg):
    import torch
    ops = torch.ops.prime_moe
    mx = dtype == "mxfp8"
    c = build_sweep_case(name, tokens, dtype, device)
    T, K, E, N, k, routing = c["cfg"]
    out = torch.zeros(T, K, dtype=torch.bfloat16, device=device)
    touched = int(c["ids_cpu"].unique().numel())
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device) if \
        touched * (N * K + K * (N // 2)) * (1 if mx else 2) < (256 << 20) else None
    flops = 3.0 * T * k * K * N
    cands = []
    for split in (True, False):
        for bn, wn in ((64, 4), (32, 8)):
            for stages in (1, 2, 3, 4):
                def cand(split=split, bn=bn, wn=wn, stages=stages):
                    s, e, n = ops.moe_align(c["ids"], E, 128, 1)
                    if not split:
                        out.zero_()
                    if mx:
                        ref_pkg.fused_moe_mxfp8(c["xq"], c["xs"], c["w1"], c["w1s"], c["w2"], c["w2s"], s, e, n, c["wts"], out, k,
                                                128, bn, wn, stages, 1, split)
                    else:
                        ref_pkg.fused_moe_bf16(c["x"], c["w1"], c["w2"], s, e, n, c["wts"], out, k, 128, bn, wn, stages, 1, 1, split)
                cands.append((cand, {"block_n": bn, "warp_n": wn, "stages": stages, "split": split}))
    best = select_knobs(cands, trial_calls=2, final_calls=5)
    if best is None:
        return {"config": name, "tokens": T, "dtype": dtype, "unavailable": "every knob setting of the reference failed"}
    ms = time_steps(best[1], 20 if flops < 5e12 else 8, flush_buf)
    del c, out, flush_buf
    torch.cuda.empty_cache()
    return {"config": name, "tokens": T, "dtype": dtype, "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "tokens_per_s": T / (ms * 1e-3), "knobs": best[2]}


def sweep_align_entry(name, device, peaks, kernel_name):
    """`moe_align` alone on the routing table of a configuration: L2 flushed before every call, achieved GB/s
    over its algorithmic bytes 4n read + 4(max_padded + max_blocks + 1) written."""
    import torch
    sys.path.insert(0, str(ROOT))
    from oracle import moe_oracle as O
    ops = torch.ops.prime_moe
    T, K, E, N, k, routing = CONFIGS[name]
    ids, _ = O.make_routing(T, E, k, 4321 + sorted(CONFIGS).index(name) + 1, routing)
    ids = ids.to(device)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    ms = time_calls(lambda: ops.moe_align(ids, E, 128, 1), 30, flush_buf)
    n = T * k
    max_padded = (n + E * 127 + 127) // 128 * 128
    nbytes = 4.0 * n + 4.0 * (max_padded + max_padded // 128 + 1)
    ach = nbytes / (ms * 1e-3) / 1e9
    del flush_buf
    torch.cuda.empty_cache()
    return {"config": name, "op": "moe_align", "n": n, "num_experts": E, "dtype": "int32", "ms_per_step": ms,
            "value": ach, "unit": "GB/s",
            "roofline": {"kernel": kernel_name, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"] + " (STREAM-style copy)",
                         "traffic": None, "algorithmic_bytes": nbytes}}


def ep_sweep_entry(name, dtype, rank, world, device, args):
    """One expert-parallel entry beside the headline of an N-GPU run: configuration 3 (DeepSeek-V3 layer, mxfp8),
    T tokens per rank, E / N experts per rank. Every rank generates only its own experts (16 at a time, seeded by
    the chunk's global index, so the layer is the same whatever N is)."""
    import torch
    sys.path.insert(0, str(ROOT))
    from oracle import moe_oracle as O
    from prime_flash_moe_b200 import capi, ep
    T, K, E, N, k, routing = CONFIGS[name]
    per = E // world
    w1q, w1s, w2q, w2s = [], [], [], []
    for e0 in range(rank * per, (rank + 1) * per, 16):
        n = min(16, (rank + 1) * per - e0)
        g = torch.Generator(device=device).manual_seed(777 + e0)
        a = torch.randn(n, N, K, device=device, generator=g, dtype=torch.bfloat16) * K ** -0.5
        b = torch.randn(n, K, N // 2, device=device, generator=g, dtype=torch.bfloat16) * (N // 2) ** -0.5
        q, sc = quantize_mx_device(a)
        w1q.append(q), w1s.append(pack_scales(sc))
        q, sc = quantize_mx_device(b)
        w2q.append(q), w2s.append(pack_scales(sc))
        del a, b
    experts = ep.LocalExperts(torch.cat(w1q), torch.cat(w2q), torch.cat(w1s), torch.cat(w2s), stages=args.stages)
    layer = ep.ExpertParallelMoE(E, experts, combine=args.ep_combine)
    g = torch.Generator(device=device).manual_seed(888 + rank)
    xq, xs = quantize_mx_device(torch.randn(T, K, device=device, generator=g).to(torch.bfloat16))
    ids, wts = O.make_routing(T, E, k, 889 + rank, routing)
    ids, wts = ids.to(device), wts.to(device)
    for _ in range(3):
        out = layer(xq, ids, wts, xs)
    barrier_sync(world)
    steps = 10
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        out = layer(xq, ids, wts, xs)
    b.record()
    barrier_sync(world)
    ms = max_over_ranks(a.elapsed_time(b), world, device) / steps
    flops = 3.0 * T * k * K * N
    phases = None
    if layer.combine_mode == "peer":
        layer.profile = True
        for _ in range(3):
            out = layer(xq, ids, wts, xs)
        phases = {k_: round(v_, 4) for k_, v_ in layer.phase_ms().items()}
    entry = {"config": name, "tokens": T, "dtype": dtype, "parallelism": f"ep{world}", "ms_per_step": ms,
             "value": world * flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "tokens_per_s": world * T / (ms * 1e-3),
             "experts_per_rank": per, "rows_computed_by_rank0": layer.last_recv_rows,
             "rows_sent_by_rank0": layer.last_sent_rows, "combine": layer.combine_mode, "phase_ms_rank0": phases,
             "finite": bool(torch.isfinite(out.float()).all()), "device_status": capi.device_status()}
    if layer.exchange is not None:
        layer.exchange.close()
    return entry


def sweep_pre_entries(device, peaks):
    """The two steps ahead of the path, at the c3 shapes (T=16384, E=256, top_k=8, K=7168): router and MX activation
    quantiser, L2 flushed before every call, achieved GB/s over their algorithmic bytes."""
    import torch
    ops = torch.ops.prime_moe
    T, K, E, N, k, _ = CONFIGS["c3"]
    g = torch.Generator(device=device).manual_seed(4400)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = []
    logits = torch.randn(T, E, device=device, generator=g)
    ms = time_calls(lambda: ops.route_topk(logits, k, True), 20, flush_buf)
    nbytes = 4.0 * T * E + 8.0 * T * k
    out.append(("route_topk", "route_topk_kernel", "fp32 logits", ms, nbytes))
    x = torch.randn(T, K, device=device, generator=g).to(torch.bfloat16)
    ms = time_calls(lambda: ops.quantize_mx(x, None), 20, flush_buf)
    nbytes = 2.0 * T * K + T * K * (1.0 + 1.0 / 32)
    out.append(("quantize_mx", "quantize_mx_kernel", "bf16 -> e4m3 + e8m0/32", ms, nbytes))
    entries = []
    for op, kernel, dtype, ms, nbytes in out:
        ach = nbytes / (ms * 1e-3) / 1e9
        entries.append({"config": "c3", "op": op, "dtype": dtype, "ms_per_step": ms, "value": ach, "unit": "GB/s",
                        "roofline": {"kernel": kernel, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                                     "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                                     "peak_source": peaks["source"] + " (STREAM-style copy)", "traffic": None,
                                     "algorithmic_bytes": nbytes}})
    del flush_buf, logits, x
    torch.cuda.empty_cache()
    return entries


SWEEP_BACKWARD = [("c0", 0), ("c2", 8192), ("c1", 0)]
BACKWARD_STEPS = (("prep", 1), ("gate_up_recompute", 2), ("d_act_swiglu", 4), ("d_w2", 8), ("d_xs", 16), ("d_w1", 32),
                  ("combine_d_x", 64))


def sweep_backward_entry(name, tokens, device, peaks):
    """Backward pass of the bf16 layer (`fused_moe_bf16_backward`; the reference has none): d_x, d_w1, d_w2 and
    d_topk_weights from d_out, L2 flushed before every call. FLOPs = 3 x forward (gate/up recompute, two dgrad and two
    wgrad GEMMs); the roofline is the tensor one over the whole call."""
    import torch
    from prime_flash_moe_b200 import capi
    ops = torch.ops.prime_moe
    c = build_sweep_case(name, tokens, "bf16", device)
    T, K, E, N, k, routing = c["cfg"]
    lib = capi.lib()
    s, e, n = ops.moe_align(c["ids"], E, 128, 1)
    d_out = torch.randn(T, K, device=device, generator=torch.Generator(device=device).manual_seed(99)).to(torch.bfloat16)
    ws = capi._workspace(lib.pmoe_fused_moe_bf16_backward_workspace_bytes(T, K, N, E, k, s.numel()), device)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    call = lambda: capi.fused_moe_bf16_backward(c["x"], c["w1"], c["w2"], d_out, s, e, n, c["wts"], k, workspace=ws)
    flops = 9.0 * T * k * K * N
    reps = 10 if flops < 2e13 else 5
    ms = time_calls(call, reps, flush_buf)
    steps = {}
    for label, bit in BACKWARD_STEPS:
        lib.pmoe_debug_set_backward_mask(bit)
        steps[label] = time_calls(call, reps, flush_buf)
    lib.pmoe_debug_set_backward_mask(127)
    call()
    # the same with the gate/up pre-activations kept by the forward call (no recompute GEMM): forward with and without
    # keeping them (one-CTA kernels, bpc = 1, both), then the backward pass fed with them
    out = torch.empty(T, K, dtype=torch.bfloat16, device=device)
    fwd_plain = time_calls(lambda: capi.fused_moe_bf16(c["x"], c["w1"], c["w2"], s, e, n, c["wts"], out, k), reps, flush_buf)
    fwd_keep = time_calls(lambda: capi.fused_moe_bf16_keep(c["x"], c["w1"], c["w2"], s, e, n, c["wts"], out, k), reps, flush_buf)
    _, gate_up = capi.fused_moe_bf16_keep(c["x"], c["w1"], c["w2"], s, e, n, c["wts"], out, k)
    ms_kept = time_calls(lambda: capi.fused_moe_bf16_backward(c["x"], c["w1"], c["w2"], d_out, s, e, n, c["wts"], k,
                                                              workspace=ws, gate_up=gate_up), reps, flush_buf)
    # ... and with the weight gradients added into fp32 tensors (a trainer's main gradients) by the wgrad epilogue
    main_grads = (torch.zeros(E, N, K, dtype=torch.float32, device=device),
                  torch.zeros(E, K, N // 2, dtype=torch.float32, device=device))
    ms_acc = time_calls(lambda: capi.fused_moe_bf16_backward(c["x"], c["w1"], c["w2"], d_out, s, e, n, c["wts"], k,
                                                             workspace=ws, gate_up=gate_up, d_w=main_grads,
                                                             accumulate=True), reps, flush_buf)
    torch.cuda.synchronize()
    assert capi.device_status() == 0, "a kernel recorded an error status"
    ach = flops / (ms * 1e-3) / 1e12
    kept = {"backward_ms": ms_kept, "forward_ms": fwd_keep, "forward_ms_without_keeping": fwd_plain,
            "tflops_over_2_thirds_of_flops": (6.0 * T * k * K * N) / (ms_kept * 1e-3) / 1e12,
            "backward_ms_accumulating_into_fp32_weight_gradients": ms_acc}
    del c, ws, d_out, flush_buf, gate_up, out, main_grads
    torch.cuda.empty_cache()
    return {"config": name, "tokens": T, "op": "backward", "dtype": "bf16", "ms_per_step": ms, "value": ach,
            "unit": "TFLOP/s", "with_kept_pre_activations": kept,
            "roofline": {"kernel": "moe_bwd_gemm_kernel (5 launches)", "bound": "tensor", "achieved": ach,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                         "peak_source": peaks["source"] + " (burst cuBLAS bf16)", "traffic": None,
                         "kernel_ms": steps}}


def run_sweep(impl, device, peaks, stages, ref_pkg=None):
    entries = []
    for name, tokens, dtype in SWEEP:
        try:
            if impl == "ours":
                entries.append(sweep_entry_ours(name, tokens, dtype, device, peaks, stages))
            else:
                entries.append(sweep_entry_reference(name, tokens, dtype, device, ref_pkg))
        except Exception as exc:            # an entry that fails is reported, not hidden
            entries.append({"config": name, "tokens": tokens, "dtype": dtype, "error": f"{type(exc).__name__}: {exc}"[:200]})
    for name in SWEEP_ALIGN:
        try:
            entries.append(sweep_align_entry(name, device, peaks, "moe_align_{hist,scan,scatter}_kernel" if impl == "ours"
                                             else "the reference's moe_align_kernel"))
        except Exception as exc:
            entries.append({"config": name, "op": "moe_align", "error": f"{type(exc).__name__}: {exc}"[:200]})
    if impl == "ours":          # the reference has no router or quantiser (it takes both from its caller)
        try:
            entries.extend(sweep_pre_entries(device, peaks))
        except Exception as exc:
            entries.append({"config": "c3", "op": "route_topk / quantize_mx", "error": f"{type(exc).__name__}: {exc}"[:200]})
        for name, tokens in SWEEP_BACKWARD:     # nor a backward pass
            try:
                entries.append(sweep_backward_entry(name, tokens, device, peaks))
            except Exception as exc:
                entries.append({"config": name, "tokens": tokens, "op": "backward",
                                "error": f"{type(exc).__name__}: {exc}"[:200]})
    return entries


def sweep_summary(entries):
    """One short string per entry for readers that keep scalar fields only."""
    parts = []
    for e in entries:
        tag = f"{e['config']}" + (f"/T{e['tokens']}" if e.get("tokens") else "") + f"/{e.get('op', e.get('dtype'))}"
        if "ms_per_step" not in e:
            parts.append(f"{tag}: failed")
            continue
        r = e.get("roofline")
        parts.append(f"{tag}: {e['ms_per_step'] * 1e3:.0f}us {e['value']:.0f}{e['unit']}" +
                     (f" {r['bound']} frac {r['frac']:.2f}" if r else ""))
    return "; ".join(parts)


# ------------------------------------------------------------------------------------------------
# arms
# ------------------------------------------------------------------------------------------------
def run_gpu_arm(args, impl):
    import torch
    world, rank, local = dist_setup(args)
    if impl == "reference" and rank != 0:
        return                     # the reference arm is single-GPU: rank 0 alone runs and prints
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        bind_to_gpu_numa_node(local)
    cfg = list(CONFIGS[args.config])
    if args.tokens:
        cfg[0] = args.tokens
    T, K, E, N, k, routing = cfg
    mx = args.dtype == "mxfp8"
    ep_mode = impl == "ours" and args.parallel == "ep"
    x, w1, w2, ids_cpu, wts_cpu = make_inputs(cfg, 1234 + rank, device, weights=not ep_mode)
    ids, wts = ids_cpu.to(device), wts_cpu.to(device)
    out = torch.zeros(T, K, dtype=torch.bfloat16, device=device)
    flops = 3.0 * T * k * K * N
    if mx:
        # OCP-MX operands computed from the bf16 tensors: e4m3 values + e8m0 scale per 32 K-elements
        xq, xs = quantize_mx_device(x)
        if not ep_mode:
            w1q, w1s = quantize_mx_weights(w1)
            w2q, w2s = quantize_mx_weights(w2)
            w1s, w2s = pack_scales(w1s), pack_scales(w2s)

    xin = (xq, xs) if mx else x      # what a step consumes as its activation input
    if ep_mode:
        # expert parallel: every rank generated the SAME full weights (seed 99), keeps its E/world experts,
        # and runs its own T tokens; dispatch / combine are NCCL all-to-alls (prime_flash_moe_b200/ep.py)
        sys.path.insert(0, str(ROOT))
        import prime_flash_moe_b200  # noqa: F401
        from prime_flash_moe_b200 import capi, ep
        gw = torch.Generator(device=device).manual_seed(99)
        w1 = torch.randn(E, N, K, device=device, generator=gw, dtype=torch.bfloat16) * K ** -0.5
        w2 = torch.randn(E, K, N // 2, device=device, generator=gw, dtype=torch.bfloat16) * (N // 2) ** -0.5
        if mx:
            w1q, w1s = quantize_mx_weights(ep.shard_experts(w1, rank, world))
            w2q, w2s = quantize_mx_weights(ep.shard_experts(w2, rank, world))
            experts = ep.LocalExperts(w1q, w2q, pack_scales(w1s), pack_scales(w2s), stages=args.stages)
        else:
            experts = ep.LocalExperts(ep.shard_experts(w1, rank, world), ep.shard_experts(w2, rank, world),
                                      stages=args.stages)
        # correctness figure carried by every expert-parallel line: the first 64 tokens of this rank through the plain
        # single-GPU operator on the FULL weights, compared below with the same rows of the expert-parallel result
        ops = torch.ops.prime_moe
        np_ = min(64, T)
        par_ref = torch.empty(np_, K, dtype=torch.bfloat16, device=device)
        ps, pe, pn = ops.moe_align(ids[:np_].contiguous(), E, 128, 1)
        if mx:
            fw1q, fw1s = quantize_mx_weights(w1)
            fw2q, fw2s = quantize_mx_weights(w2)
            ops.fused_moe_mxfp8(xq[:np_].contiguous(), xs[:np_].contiguous(), fw1q, pack_scales(fw1s), fw2q, pack_scales(fw2s),
                                ps, pe, pn, wts[:np_].contiguous().view(-1), par_ref, k, 128, 64, 4, args.stages, 1, True)
            del fw1q, fw1s, fw2q, fw2s
        else:
            ops.fused_moe_bf16(x[:np_].contiguous(), w1, w2, ps, pe, pn, wts[:np_].contiguous().view(-1), par_ref, k, 128, 64,
                               4, args.stages, 1, 1, True)
        torch.cuda.synchronize()
        del w1, w2
        torch.cuda.empty_cache()
        layer = ep.ExpertParallelMoE(E, experts, combine=args.ep_combine)
        launches_per_step = None
        ep_rows = []

        def step(x_, ids_, wts_, out_):
            if mx:
                out_.copy_(layer(x_[0], ids_, wts_, x_[1]))
            else:
                out_.copy_(layer(x_, ids_, wts_))
        knobs = {"stages": args.stages, "split": True, "experts_per_rank": E // world}
    elif impl == "ours":
        sys.path.insert(0, str(ROOT))
        import prime_flash_moe_b200  # noqa: F401
        from prime_flash_moe_b200 import capi
        ops = torch.ops.prime_moe
        (bn, wn), stages, split, bpc = ((64, 4) if args.warp_n == 4 else (32, 8)), args.stages, bool(args.split), args.bpc
        # align kernels + gather, gate/up|fused, down|finalize (+ pair classification and the two tail launches, bpc=2)
        # moe_align (one CTA up to 4096 ids, or 16384 with <= 256 experts; else histogram + scatter) + row gather,
        # gate/up|fused, down|finalize (+ pair classification and the two tail launches, bpc=2)
        align_launches = 1 if (T * k <= 4096 or (T * k <= 16384 and E <= 256)) else 2
        launches_per_step = align_launches + 3 + (3 if (bpc == 2 and split and not mx) else 0)

        def step(x_, ids_, wts_, out_):
            s, e, n = ops.moe_align(ids_, E, 128, bpc)
            if not split:
                out_.zero_()
            if mx:
                ops.fused_moe_mxfp8(x_[0], x_[1], w1q, w1s, w2q, w2s, s, e, n, wts_, out_, k, 128, bn, wn, stages, bpc,
                                    split)
            else:
                ops.fused_moe_bf16(x_, w1, w2, s, e, n, wts_, out_, k, 128, bn, wn, stages, bpc, 1, split)
        knobs = {"block_n": bn, "warp_n": wn, "stages": stages, "split": split, "bpc": bpc}
    else:
        ref_dir = ROOT / "baseline" / "_ref"
        if not (ref_dir / "prime_moe").exists():
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/prime_moe is not installed"}))
            return
        sys.path.insert(0, str(ref_dir))           # ahead of the repo root, which holds a shim of the same name
        import prime_moe as ref_pkg
        assert str(ref_dir) in str(Path(ref_pkg.__file__).resolve()), "wrong prime_moe imported"
        ops = torch.ops.prime_moe
        launches_per_step = None
        cands = []
        for split in (True, False):
            for bn, wn in ((64, 4), (32, 8)):
                for stages in (1, 2, 3, 4):
                    def cand(x_, ids_, wts_, out_, split=split, bn=bn, wn=wn, stages=stages):
                        s, e, n = ops.moe_align(ids_, E, 128, 1)
                        if not split:
                            out_.zero_()
                        if mx:
                            ref_pkg.fused_moe_mxfp8(x_[0], x_[1], w1q, w1s, w2q, w2s, s, e, n, wts_, out_, k, 128, bn,
                                                    wn, stages, 1, split)
                        else:
                            ref_pkg.fused_moe_bf16(x_, w1, w2, s, e, n, wts_, out_, k, 128, bn, wn, stages, 1, 1, split)
                    cands.append((lambda cand=cand: cand(xin, ids, wts, out),
                                  {"block_n": bn, "warp_n": wn, "stages": stages, "split": split, "bpc": 1, "_step": cand}))
        best = select_knobs(cands)
        if best is None:
            print(json.dumps({"impl": "reference", "unavailable": "every knob setting of the reference failed"}))
            return
        knobs = dict(best[2])
        step = knobs.pop("_step")
        torch.cuda.synchronize()
        time.sleep(0.5)       # the knob sweep ran ~150 back-to-back steps: let the power state settle before timing

    ref_world = 1 if impl == "reference" else world
    # bytes of the weights one step reads: experts actually routed to x (w1 + w2)
    touched_weight_bytes = int(ids_cpu.unique().numel()) * (N * K + K * (N // 2)) * (1 if mx else 2)
    flush_l2 = touched_weight_bytes < (256 << 20)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device) if flush_l2 else None
    # ---- device-resident timing ----
    for _ in range(max(args.warmup, 3)):
        step(xin, ids, wts, out)
    barrier_sync(ref_world)
    ep_fallback = None
    if ep_mode and layer.combine_mode == "peer":
        # the peer-memory exchange has bounded waits: if any rank recorded an expired one during warm-up (a peer that
        # cannot be reached, a rank far behind), every rank switches to the NCCL exchange together instead of timing
        # a broken step
        st = max_over_ranks(float(capi.device_status()), world, device)
        if st != 0:
            capi.reset_device_status()
            ep_fallback = f"device status {int(st)} after warm-up in peer mode: switched to the NCCL exchange"
            if layer.exchange is not None:
                layer.exchange.close()
            layer = ep.ExpertParallelMoE(E, experts, combine="nccl")
            for _ in range(3):
                step(xin, ids, wts, out)
            barrier_sync(ref_world)
    with ClockSampler(local) as clocks:
        if flush_l2:
            # the weights a step touches would stay in the 126 MB L2 from one step to the next: write a 256 MB
            # buffer between steps and time every step with its own pair of events (the flush is not timed)
            pairs = []
            for _ in range(args.steps):
                flush_buf.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                step(xin, ids, wts, out)
                b.record()
                pairs.append((a, b))
            barrier_sync(ref_world)
            ms_total = max_over_ranks(sum(a.elapsed_time(b) for a, b in pairs), ref_world, device)
        else:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                step(xin, ids, wts, out)
            b.record()
            barrier_sync(ref_world)
            ms_total = max_over_ranks(a.elapsed_time(b), ref_world, device)
    ms_step = ms_total / args.steps
    value = ref_world * flops / (ms_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel: timed alone, right after the device-resident loop (same thermal state),
    # with the SM clock sampled while it runs ----
    peaks = measured_peaks()
    roofline = None
    roof_clocks = ClockSampler(local)
    roof_clocks.__enter__()
    if impl == "ours" and args.split and mx and not ep_mode:
        roofline = roofline_mxfp8(args, capi, ops, (xq, xs, w1q, w1s, w2q, w2s), ids, wts, out, cfg, peaks, value / world,
                                  flush_buf if flush_l2 else None)
        roofline = weight_streaming_roofline(roofline, cfg, ids, roofline["kernel_ms"]["moe_up_mxfp8"], ms_step, peaks, True,
                                             431.8e6 if (args.config == "c2" and args.tokens == 128) else None)
    if impl == "ours" and args.split and not mx and not ep_mode:
        # dominant kernel = the gate/up GEMM (2/3 of the FLOPs); timed alone through the profiling hook
        lib = capi.lib()
        step(x, ids, wts, out)                      # fills the workspace-independent state
        s, e, n = ops.moe_align(ids, E, 128, args.bpc)
        nbytes = lib.pmoe_fused_moe_bf16_workspace_bytes(T, K, N, s.numel(), 1)
        ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        off = (-ws.data_ptr()) % 1024
        ws = ws[off:off + nbytes]
        call = lambda: capi.fused_moe_bf16(x, w1, w2, s, e, n, wts, out, k, 128, 64 if args.warp_n == 4 else 32, args.warp_n,
                                           args.stages, args.bpc, 1, True, workspace=ws)
        call()
        per_kernel = {}
        masks = [("gather_rows", 1), ("moe_up_bf16", 2), ("moe_down_bf16", 4)]
        if args.bpc == 2:      # the CTA-pair kernels without the single-block tail launches that follow them
            masks = [("gather_rows", 1), ("moe_up_bf16", 2 | 8), ("moe_up_bf16_with_tails", 2), ("moe_down_bf16", 4 | 8),
                     ("moe_down_bf16_with_tails", 4)]
        for name, mask in masks:
            lib.pmoe_debug_set_phase_mask(mask)
            per_kernel[name] = time_calls(call, 20, flush_buf if flush_l2 else None)
        lib.pmoe_debug_set_phase_mask(7)
        call()
        torch.cuda.synchronize()
        rows_dominant = T * k
        if args.bpc == 2 and os.environ.get("PMOE_PAIR_TAILS", "1") != "0":
            # rows of the half-empty last pairs run on the one-CTA kernels, not on the kernel timed here
            cnt = torch.bincount(ids_cpu.reshape(-1).long(), minlength=E)
            rem = cnt % 256
            rows_dominant -= int(rem[(rem > 0) & (rem <= 128)].sum())
        up_flops = 2.0 * rows_dominant * K * N
        achieved = up_flops / (per_kernel["moe_up_bf16"] * 1e-3) / 1e12
        # DRAM bytes of one launch of that kernel, from the ncu captures summarised under profiles/
        traffic = {("c1", 2): 2.713e9, ("c2", 1): 1.112e9}.get((args.config, args.bpc)) \
            if (not args.tokens and args.stages == 4 and args.warp_n == 4) else None
        roofline = {"kernel": "moe_pair_bf16_kernel<up>" if args.bpc == 2 else "moe_up_bf16_kernel", "bound": "tensor",
                    "rows": rows_dominant, "achieved": achieved,
                    "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                    "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                    "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
                    "traffic": traffic, "algorithmic_bytes": float(E * N * K * 2 + rows_dominant * K * 2 + rows_dominant * N + T * K * 2),
                    "kernel_ms": per_kernel, "whole_op_frac": value / world / peaks["bf16_tflops"]}
        roofline = weight_streaming_roofline(roofline, cfg, ids, per_kernel["moe_up_bf16"], ms_step, peaks, False,
                                             835.3e6 if (args.config == "c2" and args.tokens == 128) else None)
        assert capi.device_status() == 0, "a kernel recorded an error status"
    roof_clocks.__exit__(None, None, None)
    if roofline is not None:
        roofline["sm_mhz_during_kernel_timing"] = roof_clocks.summary()["sm_mhz"]

    # ---- end to end: host buffers, copies inside the timed region ----
    # What a caller feeding the layer from host memory does: two sets of device buffers, the H2D copy of step
    # i+1 and the D2H copy of step i-1 run on their own streams beside the kernels of step i. Every step's inputs
    # come from pinned host memory and every step's result is read back to pinned host memory.
    hx = tuple(t.cpu().pin_memory() for t in xin) if mx else (x.cpu().pin_memory(),)
    hids, hwts = ids_cpu.pin_memory(), wts_cpu.pin_memory()
    houts = [torch.empty(T, K, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dxs = [tuple(torch.empty_like(t, device=device) for t in hx) for _ in range(2)]
    didss, dwtss = [torch.empty_like(ids) for _ in range(2)], [torch.empty_like(wts) for _ in range(2)]
    outs = [torch.empty_like(out) for _ in range(2)]
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()

    def e2e_run(n):
        in_done, comp_done, out_done = {}, {}, {}
        for i in range(n):
            j = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(comp_done[i - 2])            # the kernels of step i-2 are done with buffer j
                for d_, h_ in zip(dxs[j], hx):
                    d_.copy_(h_, non_blocking=True)
                didss[j].copy_(hids, non_blocking=True)
                dwtss[j].copy_(hwts, non_blocking=True)
                in_done[i] = s_in.record_event()
            s_main.wait_event(in_done[i])
            if i >= 2:
                s_main.wait_event(out_done[i - 2])               # result buffer j has been read back
            step(dxs[j] if mx else dxs[j][0], didss[j], dwtss[j], outs[j])
            comp_done[i] = s_main.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[i])
                houts[j].copy_(outs[j], non_blocking=True)
                out_done[i] = s_out.record_event()
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    # at least 50 steps: the first step's H2D copy and the last step's D2H copy cannot hide behind a neighbouring step's
    # kernels, and over 20 steps of 2.4 ms that pipeline fill / drain alone is ~5 % of the measurement
    e2e_steps = min(max(args.steps, 50), 200)
    e2e_run(3)
    e2e_runs = []
    for _ in range(2):      # two timed regions, the faster one is reported (both arms alike): on a fresh box the first
        barrier_sync(ref_world)   # region through host memory now and then runs at half speed for either arm
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        e2e_run(e2e_steps)
        b.record()
        barrier_sync(ref_world)
        e2e_runs.append(max_over_ranks(a.elapsed_time(b), ref_world, device) / e2e_steps)
    e2e_ms = min(e2e_runs)
    hout = houts[0]
    h2d = sum(t.numel() * t.element_size() for t in hx) + hids.numel() * 4 + hwts.numel() * 4
    d2h = hout.numel() * 2
    e2e = {"value": ref_world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
           "ms_per_step_of_both_regions": e2e_runs}

    cpu_baseline = None
    if rank == 0 and not args.no_cpu_baseline and not ep_mode and ref_world == 1:
        sample = 256 if T >= 256 else T
        tf, secs, threads = time_cpu_oracle(x, w1, w2, ids_cpu, wts_cpu, sample)
        cpu_baseline = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"first {sample} of {T} tokens of the same batch, torch CPU grouped_mm oracle, "
                                  f"{secs:.2f} s", "host_cpus": os.cpu_count()}

    ep_parity = None
    if ep_mode:
        # kernels of this package per step: plan (3) + moe_align (1 or 3) + row gather, gate/up, down (3) + combine (1)
        step(xin, ids, wts, out)
        torch.cuda.synchronize()
        ep_rows.append(layer.last_recv_rows)
        ep_phases = None
        if layer.combine_mode == "peer":      # phase times of five more steps (CUDA events on this rank's stream)
            layer.profile = True
            for _ in range(5):
                step(xin, ids, wts, out)
            ep_phases = {k_: round(v_, 4) for k_, v_ in layer.phase_ms().items()}
            layer.profile = False
        # plan (3) + moe_align (1 or 2) + row gather, gate/up, down (3) + combine (1) (+ publish, push, 2 signals,
        # prepare, return: 6 in peer mode)
        n_local = (world * T if layer.combine_mode == "peer" else ep_rows[-1]) * k      # ids moe_align sees on this rank
        align_launches = 1 if (n_local <= 4096 or (n_local <= 16384 and E // world <= 256)) else 2
        launches_per_step = 3 + align_launches + 3 + 1 + (6 if layer.combine_mode == "peer" else 0)
        a_, b_ = out[:np_].float(), par_ref.float()
        ep_parity = max_over_ranks(float((a_ - b_).abs().max() / b_.abs().max().clamp_min(1e-30)), world, device)
    ep_info = None
    if ep_mode:
        ep_info = {"rows_computed_by_rank0_last_step": ep_rows[-1] if ep_rows else None,
                   "rows_sent_by_rank0_last_step": layer.last_sent_rows, "routes_per_rank": T * k,
                   "tokens_per_rank": T,
                   "parity": ep_parity,
                   "parity_what": "max over ranks of max|ep_out - single_gpu_out| / max|single_gpu_out| on each "
                                  "rank's first 64 tokens (single-GPU operator on the full weights)",
                   "combine": layer.combine_mode, "fallback": ep_fallback, "phase_ms_rank0": ep_phases,
                   "collective": ("none on the data path: rows, slot tables, counts and partial sums are stored "
                                  "into the peers' buffers over NVLink by this library's kernels"
                                  if layer.combine_mode == "peer" else
                                  "NCCL all-to-all (dispatch + combine)") + ", one row per (token, rank) visit"}
        if layer.exchange is not None:
            layer.exchange.close()
            layer.exchange = None

    sweep = None
    default_run = (args.config == "c1" and not args.tokens and args.dtype == "bf16" and args.split and world == 1)
    if default_run and not args.no_sweep:
        # the other configurations, after the headline's tensors are gone
        x = w1 = w2 = xin = out = outs = dxs = houts = hx = flush_buf = None
        if impl == "ours":
            ws = call = None
        torch.cuda.empty_cache()
        sweep = run_sweep(impl, device, peaks, args.stages, ref_pkg if impl == "reference" else None)
    elif ep_mode and not args.no_sweep and args.config == "c1" and CONFIGS["c3"][2] % world == 0:
        x = xin = out = outs = dxs = houts = hx = flush_buf = layer = experts = None
        torch.cuda.empty_cache()
        sweep = [ep_sweep_entry("c3", "mxfp8", rank, world, device, args)]

    if rank == 0:
        line = {
            "metric": "moe_ffn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": ref_world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "mxfp8 (e4m3 x e8m0/32, fp32 accumulate)" if mx else "bf16",
            "data": "synthetic", "tokens_per_s": ref_world * T / (ms_step * 1e-3),
            "config": {"workload": f"{args.config}: T={T} K={K} E={E} N={N} top_k={k} routing={routing} "
                                   f"(per GPU), moe_align + fused_moe_{args.dtype}",
                       "knobs": knobs, "parallelism": f"{args.parallel}{ref_world}",
                       "l2": (f"a step touches {touched_weight_bytes / 1e6:.0f} MB of weights: L2 flushed (256 MB "
                              "written) between steps, every step timed with its own events") if flush_l2 else
                             (f"a step reads {touched_weight_bytes / 1e6:.0f} MB of weights, more than the 126 MB L2: "
                              "no flush between steps")},
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": (launches_per_step or 0) * args.steps,
            "roofline": roofline, "cpu_baseline": cpu_baseline,
        }
        if ep_mode:
            line["config"]["ep"] = ep_info
        if impl == "reference":
            line["impl"] = "reference"
            line["gpu_launches"] = None
        line["clocks"]["ms_per_step_x_sm_mhz"] = (ms_step * line["clocks"]["sm_mhz"]) if line["clocks"]["sm_mhz"] else None
        if sweep is not None:
            line["config"]["sweep"] = sweep_summary(sweep)
            line["sweep"] = sweep          # last key of the line
        print(json.dumps(line))


def run_cpu_arm(args):
    """`--impl cpu`: the reference's PyTorch MoE (oracle port) on the host cores, bounded sample."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, str(ROOT))
    cfg = list(CONFIGS[args.config])
    if args.tokens:
        cfg[0] = args.tokens
    T, K, E, N, k, routing = cfg
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    x, w1, w2, ids, wts = make_inputs(cfg, 1234, dev)
    sample = min(T, 256)
    vals = []
    for _ in range(max(1, min(args.steps, 3))):
        tf, secs, threads = time_cpu_oracle(x, w1, w2, ids, wts, sample)
        vals.append((tf, secs))
    tf, secs = max(vals)
    cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
           "sample": f"first {sample} of {T} tokens, torch CPU grouped_mm oracle"}
    print(json.dumps({"impl": "cpu", "metric": "moe_ffn_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 0,
                      "steps": len(vals), "warmup": 1, "ms_per_step": secs * 1e3, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"{args.config}: T={T} K={K} E={E} N={N} top_k={k} (sample {sample} tokens)"},
                      "cpu_baseline": cpu,
                      "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_align_only(args):
    """`--op moe_align`: the routing kernels alone (a few MB of traffic; the command the ncu summary of these
    kernels under profiles/ was made with)."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    sys.path.insert(0, str(ROOT))
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import prime_moe  # noqa: F401
        name = "the reference's moe_align_kernel"
    else:
        import prime_flash_moe_b200  # noqa: F401
        name = "moe_align_{hist,scan,scatter}_kernel"
    e = sweep_align_entry(args.config, device, measured_peaks(), name)
    e.update({"metric": "moe_align_gbs", "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
              "impl": args.impl})
    print(json.dumps(e))


def run_pre_only(args):
    """`--op pre`: router and MX activation quantiser alone (the command their ncu summary under profiles/ was made
    with). One JSON line per kernel."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    sys.path.insert(0, str(ROOT))
    import prime_flash_moe_b200  # noqa: F401
    for e in sweep_pre_entries(device, measured_peaks()):
        e.update({"metric": e["op"] + "_gbs", "n_gpus": 1, "higher_is_better": True, "data": "synthetic", "impl": "ours"})
        print(json.dumps(e))


def run_backward_only(args):
    """`--op backward`: the bf16 backward pass alone on --config (--tokens overrides T). One JSON line."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    sys.path.insert(0, str(ROOT))
    import prime_flash_moe_b200  # noqa: F401
    e = sweep_backward_entry(args.config, args.tokens or 0, device, measured_peaks())
    e.update({"metric": "moe_ffn_backward_tflops", "n_gpus": 1, "higher_is_better": True, "data": "synthetic", "impl": "ours"})
    print(json.dumps(e))


def run_train_only(args):
    """`--op train`: one training step of the bf16 layer on --config - forward that keeps the gate/up
    pre-activations + backward (9·T·k·K·N FLOPs per rank). One GPU: the autograd layer `moe_ffn`; under torchrun: the
    expert-parallel layer's `forward_train` (E / N experts and T tokens per rank, NCCL exchange). Timed with CUDA
    events over --steps steps after --warmup, max over ranks; one JSON line from rank 0."""
    import torch
    world, rank, local = dist_setup(args)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    sys.path.insert(0, str(ROOT))
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi, ep
    T, K, E, N, k, routing = CONFIGS[args.config]
    if args.tokens:
        T = args.tokens
    assert E % world == 0, "the experts must divide over the ranks"
    per = E // world
    g = torch.Generator(device=device).manual_seed(7000 + rank)
    x = torch.randn(T, K, device=device, generator=g).to(torch.bfloat16).requires_grad_(True)
    d_out = torch.randn(T, K, device=device, generator=g).to(torch.bfloat16)
    gw = torch.Generator(device=device).manual_seed(7100 + rank)          # this rank's experts only
    w1 = (torch.randn(per, N, K, device=device, generator=gw, dtype=torch.bfloat16) * K ** -0.5).requires_grad_(True)
    w2 = (torch.randn(per, K, N // 2, device=device, generator=gw, dtype=torch.bfloat16) * (N // 2) ** -0.5).requires_grad_(True)
    from oracle import moe_oracle as O
    ids, wts = O.make_routing(T, E, k, 7200 + rank, routing)
    ids, wts = ids.to(device), wts.to(device).requires_grad_(True)
    if world > 1:
        layer = ep.ExpertParallelMoE(E, ep.LocalExperts(w1, w2), combine="nccl")
        fwd = lambda: layer.forward_train(x, ids, wts)
    else:
        fwd = lambda: P.moe_ffn(x, w1, w2, ids, wts)

    def step():
        for t in (x, w1, w2, wts):
            t.grad = None
        fwd().backward(d_out)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier_sync(world)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    barrier_sync(world)
    ms = max_over_ranks(a.elapsed_time(b) / args.steps, world, device)
    assert capi.device_status() == 0, "a kernel recorded an error status"
    if rank == 0:
        flops = 9.0 * T * k * K * N * world
        print(json.dumps({"metric": "moe_ffn_train_step_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
                          "impl": "ours", "tokens_per_s": T * world / (ms * 1e-3),
                          "config": {"workload": args.config, "tokens_per_rank": T, "experts_per_rank": per,
                                     "parallelism": f"ep{world}" if world > 1 else "single",
                                     "exchange": "nccl all-to-all" if world > 1 else None,
                                     "flops": "forward 3·T·k·K·N + backward 6·T·k·K·N (pre-activations kept)"}}))


def main():
    args = parse_args()
    if args.bpc == 0:
        # CTA pairs pay off on wide layers (measured: c1 N=28672 +6 %); narrow ones run best on the one-CTA
        # kernels with the in-kernel LSU gather (c2 N=1536 +5 %)
        args.bpc = 2 if (args.dtype == "bf16" and args.split and CONFIGS[args.config][3] >= 8192) else 1
    if args.parallel == "auto":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        args.parallel = "ep" if world > 1 and CONFIGS[args.config][2] % world == 0 else "replica"
    if args.op == "moe_align":
        run_align_only(args)
    elif args.op == "pre":
        run_pre_only(args)
    elif args.op == "backward":
        run_backward_only(args)
    elif args.op == "train":
        run_train_only(args)
    elif args.impl == "cpu":
        run_cpu_arm(args)
    else:
        run_gpu_arm(args, args.impl)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
