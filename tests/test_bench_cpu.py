"""Host-side pieces of bench.py that need no GPU: its OCP-MX quantiser and scale packing (they prepare the mxfp8
inputs of BOTH benchmark arms) against the oracle, the sweep list against the benchmark configurations, and the
one-string sweep summary."""
import importlib.util
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("_pmoe_bench", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_bench_quantiser_and_packing_match_the_oracle():
    from oracle import moe_oracle as O
    b = _bench()
    g = torch.Generator().manual_seed(3)
    t = torch.randn(3, 256, 128, generator=g).to(torch.bfloat16)
    t[0, 0, :32] = 0
    q, s = b.quantize_mx_device(t)
    q2, s2 = O.quantize_mx(t)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s.view(torch.uint8), s2.view(torch.uint8))
    qc, sc = b.quantize_mx_weights(t, chunk=2)
    assert torch.equal(qc.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(sc.view(torch.uint8), s2.view(torch.uint8))
    assert torch.equal(b.pack_scales(s).view(torch.uint8), O.pack_scales_blocked(s).view(torch.uint8))


def test_sweep_covers_the_benchmark_configurations():
    b = _bench()
    assert set(b.CONFIGS) >= {"c0", "c1", "c2", "c3", "c4"}
    assert b.CONFIGS["c1"] == (4096, 4096, 8, 28672, 2, "uniform")
    assert b.CONFIGS["c3"] == (16384, 7168, 256, 4096, 8, "uniform")
    assert b.CONFIGS["c4"][:5] == (65536, 4096, 128, 3072, 8) and b.CONFIGS["c4"][5] == "zipf"
    names = {(c, d) for c, _, d in b.SWEEP}
    assert ("c3", "mxfp8") in names and ("c4", "bf16") in names and ("c4", "mxfp8") in names and ("c0", "bf16") in names
    assert {t for c, t, _ in b.SWEEP if c == "c2"} == {16, 128, 8192}
    assert b.SWEEP_ALIGN == ["c4", "c3"]
    assert ("c1", 0) in b.SWEEP_BACKWARD and ("c2", 8192) in b.SWEEP_BACKWARD        # backward pass beside the forward sweep
    assert sum(bit for _, bit in b.BACKWARD_STEPS) == 127                              # every step of the mask, once


def test_operations_the_bench_can_time(monkeypatch):
    b = _bench()
    for op in ("moe", "moe_align", "pre", "backward", "train"):
        monkeypatch.setattr("sys.argv", ["bench.py", "--op", op])
        assert b.parse_args().op == op


def test_sweep_summary_is_one_string_per_entry():
    b = _bench()
    entries = [
        {"config": "c2", "tokens": 8192, "dtype": "mxfp8", "ms_per_step": 0.44, "value": 1400.0, "unit": "TFLOP/s",
         "roofline": {"bound": "tensor", "frac": 0.58}},
        {"config": "c4", "op": "moe_align", "ms_per_step": 0.03, "value": 140.0, "unit": "GB/s",
         "roofline": {"bound": "hbm", "frac": 0.02}},
        {"config": "c3", "tokens": 0, "dtype": "mxfp8", "error": "RuntimeError: x"},
    ]
    text = b.sweep_summary(entries)
    assert text.count(";") == 2
    assert "c2/T8192/mxfp8: 440us 1400TFLOP/s tensor frac 0.58" in text
    assert "c4/moe_align: 30us 140GB/s hbm frac 0.02" in text and "c3/mxfp8: failed" in text
