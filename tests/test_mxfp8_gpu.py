"""fused_moe_mxfp8 on the GPU against the CPU oracle, the golden vectors and the reference's kernels.

Tolerances: max|out - ref| <= 2e-2 * max|ref| against the requant-aware dequantised fp32 oracle (the MX
re-quantisation of the activation applied to the fp32 SwiGLU value, as the kernels do), and the stated
looser bound 1e-1 * max|ref| against the dequantised fp32 oracle WITHOUT activation re-quantisation;
plus the reference's own gates rel_clamp_10 <= 0.002, rel_clamp_1 <= 0.02 (test/test_mxfp8.py:14-15) on
its own input distribution."""
import pytest
import torch

from oracle import moe_oracle as O, ref_kernels as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2
TOL_NO_REQUANT = 1e-1


def quantised_case(T, K, E, N, k, seed, **kw):
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed, **kw)
    q = {"x": O.quantize_mx(x), "w1": O.quantize_mx(w1), "w2": O.quantize_mx(w2)}
    deq = {n: O.dequantize_mx(*q[n]) for n in q}
    return q, deq, ids, wts


def run_mine(q, ids, wts, split, stages=4, bn=64, wn=4, via="capi", bpc=1):
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    (xq, xs), (w1q, w1s), (w2q, w2s) = q["x"], q["w1"], q["w2"]
    E = w1q.shape[0]
    T, K = xq.shape
    k = ids.shape[1]
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, bpc)
    out = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV) if not split else \
        torch.full((T, K), float("nan"), dtype=torch.bfloat16, device=DEV)
    args = (xq.to(DEV), xs.to(DEV), w1q.to(DEV), P.pack_scales_blocked(w1s).to(DEV), w2q.to(DEV),
            P.pack_scales_blocked(w2s).to(DEV), s, e, n, wts.to(DEV), out, k, 128, bn, wn, stages, bpc, split)
    if via == "capi":
        capi.fused_moe_mxfp8(*args)
    else:
        assert P.fused_moe_mxfp8(*args) is out
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    return out.cpu(), args


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("T,K,E,N,k", [
    (1, 256, 2, 256, 1), (8, 256, 1, 256, 1), (64, 512, 4, 512, 2), (130, 256, 5, 768, 3),
    (256, 4096, 8, 512, 4),          # benchmark configuration 0 shape, mxfp8 operands
    (128, 2048, 128, 1536, 8),       # Qwen3-30B-A3B layer, T=128
    (300, 1024, 8, 1024, 4),
])
def test_vs_fp32_oracle(T, K, E, N, k, split):
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=T + K)
    out, _ = run_mine(q, ids, wts, split)
    assert torch.isfinite(out.float()).all()
    ref_rq = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    ref_nq = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=False)
    assert O.max_rel_to_peak(out, ref_rq) <= TOL
    assert O.max_rel_to_peak(out, ref_nq) <= TOL_NO_REQUANT


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("bn,wn", [(64, 4), (32, 8)])
@pytest.mark.parametrize("stages", [1, 2, 3, 4])
def test_knobs(split, bn, wn, stages):
    q, deq, ids, wts = quantised_case(200, 512, 6, 512, 3, seed=stages)
    ref = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    out, _ = run_mine(q, ids, wts, split, stages=stages, bn=bn, wn=wn, via="torch")
    assert O.max_rel_to_peak(out, ref) <= TOL


def test_golden_vectors(golden):
    """Output of the reference's mxfp8 test oracle (test/test_mxfp8.py:50-77) stored in tests/golden. That
    oracle rounds the activation to bf16 before re-quantising it, the kernels (the reference's too)
    re-quantise the fp32 value, which flips a few e4m3 roundings: bound 5e-2 of the peak."""
    f8, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    for case in golden["moe_mxfp8"]:
        q = {"x": (case["x_q"].view(f8), case["x_scales"].view(e8)),
             "w1": (case["w1_q"].view(f8), case["w1_scales"].view(e8)),
             "w2": (case["w2_q"].view(f8), case["w2_scales"].view(e8))}
        for split in (True, False):
            out, _ = run_mine(q, case["topk_ids"], case["topk_weights"], split)
            assert O.max_rel_to_peak(out, case["out"]) <= 5e-2


@pytest.mark.parametrize("T", [8, 32, 128, 256])
@pytest.mark.parametrize("E,N,K", [(8, 256, 4096), (37, 512, 4096), (257, 256, 7168)])
def test_reference_sweep_distribution(T, E, N, K):
    """Inputs, routing and gates of the reference's mxfp8 sweep (test/test_mxfp8.py:112-199)."""
    g = torch.Generator().manual_seed(T * 1000 + E)
    x = (torch.randn(T, K, generator=g) * 0.05).to(torch.bfloat16)
    w1 = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, K, N // 2, generator=g) * 0.05).to(torch.bfloat16)
    q = {"x": O.quantize_mx(x), "w1": O.quantize_mx(w1), "w2": O.quantize_mx(w2)}
    ids = torch.randint(0, E - 1, (T, 9), generator=g, dtype=torch.int32)
    ids[:, -1] = E - 1
    wts = torch.softmax(torch.randn(T, 9, generator=g), dim=-1)
    deq = {n: O.dequantize_mx(*q[n]).to(torch.bfloat16) for n in q}
    ref = O.moe_ref_bf16(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    for split, (bn, wn), stages in ((False, (32, 8), 1), (False, (64, 4), 2), (True, (64, 4), 4)):
        out, _ = run_mine(q, ids, wts, split, stages=stages, bn=bn, wn=wn)
        assert torch.isfinite(out.float()).all()
        assert O.rel_clamp(out, ref, 10.0) <= 0.002
        assert O.rel_clamp(out, ref, 1.0) <= 0.02


def test_public_wrapper_matches_raw_operator():
    """The wrapper returns `out` and agrees with the raw op (test/test_mxfp8.py:203-239)."""
    import prime_flash_moe_b200 as P
    q, deq, ids, wts = quantised_case(128, 4096, 8, 256, 4, seed=77, x_std=0.05, w_std=0.05)
    out, args = run_mine(q, ids, wts, False, stages=1, bn=32, wn=8, via="torch")
    raw = torch.zeros_like(args[10])
    torch.ops.prime_moe.fused_moe_mxfp8(*args[:10], raw, *args[11:])
    torch.cuda.synchronize()
    assert torch.allclose(raw.float().cpu(), out.float(), rtol=1e-2, atol=2e-3)


def test_argument_checks():
    import prime_flash_moe_b200 as P
    q, deq, ids, wts = quantised_case(16, 256, 2, 256, 2, seed=1)
    _, args = run_mine(q, ids, wts, True)
    a = list(args)

    def bad(i, v):
        b = list(a)
        b[i] = v
        with pytest.raises(RuntimeError):
            P.fused_moe_mxfp8(*b)

    bad(12, 64)           # block_m
    bad(13, 16)           # (block_n, warp_n)
    bad(15, 5)            # stages 1..4
    bad(16, 3)            # bpc is 1 or 2
    bad(16, 2)            # bpc=2 needs routing tables padded to 256 rows (these are padded to 128: 384 rows)
    bad(1, a[1][:8])      # x_scales numel
    bad(0, a[0].view(torch.uint8))    # dtype
    bad(3, a[3].view(torch.uint8))    # scale dtype


@pytest.mark.skipif(not R.available(), reason="oracle/_ref (reference kernels) not built")
@pytest.mark.parametrize("T,K,E,N,k", [(256, 4096, 8, 512, 4), (128, 2048, 128, 1536, 8), (1024, 2048, 16, 1536, 4)])
def test_vs_reference_kernels(T, K, E, N, k):
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=T)
    ref32 = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    for split in (True, False):
        mine, args = run_mine(q, ids, wts, split)
        ref_out = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
        R.fused_moe_mxfp8(*args[:10], ref_out, k, 128, 64, 4, 2, 1, split)
        torch.cuda.synchronize()
        assert O.max_rel_to_peak(mine, ref32) <= TOL
        # the reference's split=False result itself sits ~2e-2 from the oracle (bf16 atomics)
        # (the reference's bf16 atomics make its own result vary from run to run; observed distance to
        # this library 0.6e-2 .. 2.4e-2, so the bound is two tolerances to keep the check stable)
        assert O.max_rel_to_peak(mine, ref_out.cpu()) <= 2.0 * TOL


def test_full_size_properties_qwen3():
    """Qwen3-30B-A3B layer at T=8192 (benchmark configuration 2), mxfp8: finite, a 64-token slice
    reproduces the same rows, and those rows match the CPU oracle."""
    T, K, E, N, k = 8192, 2048, 128, 1536, 8
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=5)
    a, _ = run_mine(q, ids, wts, True)
    assert torch.isfinite(a.float()).all()
    sub_q = {"x": (q["x"][0][:64], q["x"][1][:64]), "w1": q["w1"], "w2": q["w2"]}
    sub, _ = run_mine(sub_q, ids[:64], wts[:64], True)
    # same arithmetic per routed row; the eight bf16 reductions into an output element land in a different order
    assert O.max_rel_to_peak(sub, a[:64]) <= TOL
    ref = O.moe_ref_fp32(deq["x"][:64], deq["w1"], deq["w2"], ids[:64], wts[:64], requant_act=True)
    assert O.max_rel_to_peak(a[:64], ref) <= TOL
    b, _ = run_mine(sub_q, ids[:64], wts[:64], False)
    assert O.max_rel_to_peak(b, ref) <= TOL


@pytest.mark.parametrize("stages", [1, 4])
@pytest.mark.parametrize("T,K,E,N,k", [(8, 256, 1, 256, 1), (300, 512, 4, 512, 2), (256, 4096, 8, 512, 4),
                                       (128, 2048, 128, 1536, 8), (2048, 2048, 32, 2048, 4), (1000, 7168, 8, 1024, 8)])
def test_two_cta_pipeline(T, K, E, N, k, stages):
    """bpc=2 (not in the reference, whose mxfp8 path is bpc=1 only): CTA pairs with tcgen05.mma.cta_group::2 on
    routing tables padded to 256 rows. Same arithmetic per output row as the one-CTA pipeline (same K order,
    same requantisation), so besides the oracle bound the two must agree up to the order of the bf16
    reductions into `out`."""
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=7 * T + K)
    ref = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    pair, _ = run_mine(q, ids, wts, True, stages=stages, bpc=2)
    assert torch.isfinite(pair.float()).all()
    assert O.max_rel_to_peak(pair, ref) <= TOL
    one, _ = run_mine(q, ids, wts, True, stages=stages, bpc=1)
    assert O.max_rel_to_peak(pair, one.float()) <= TOL


def test_two_cta_rejects_fused_pipeline():
    import prime_flash_moe_b200 as P
    q, deq, ids, wts = quantised_case(64, 256, 2, 256, 2, seed=1)
    with pytest.raises(RuntimeError):
        run_mine(q, ids, wts, False, bpc=2, via="torch")


@pytest.mark.parametrize("T,K,E,N,k", [
    (1, 256, 2, 256, 1), (1, 2048, 128, 1536, 8), (16, 2048, 128, 1536, 8), (8, 256, 1, 512, 1),
    (32, 256, 1, 256, 1), (33, 256, 1, 256, 1), (8, 7168, 4, 512, 4), (5, 512, 7, 768, 3), (200, 512, 6, 512, 3),
])
def test_short_row_blocks(T, K, E, N, k, monkeypatch):
    """Row blocks holding at most 32 routed rows load and store only those rows of the A operand and of the
    activation tile (short TMA boxes); PMOE_SHORT_A=0 moves whole 128-row tiles. Both must meet the oracle
    bound and agree with each other."""
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=3 * T + K)
    ref = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    monkeypatch.setenv("PMOE_SHORT_A", "3")
    short, _ = run_mine(q, ids, wts, True)
    monkeypatch.setenv("PMOE_SHORT_A", "0")
    full, _ = run_mine(q, ids, wts, True)
    assert torch.isfinite(short.float()).all()
    assert O.max_rel_to_peak(short, ref) <= TOL
    assert O.max_rel_to_peak(full, ref) <= TOL
    # same arithmetic per routed row; the top_k bf16 reductions into an output element land in a different order
    # from run to run (with top_k = 8 two orders differ by up to ~1.3e-2 of the peak)
    assert O.max_rel_to_peak(short, full.float()) <= TOL


def test_ex_entry_point_live_rows():
    """`pmoe_fused_moe_mxfp8_ex`: worst-case sized buffers with only the leading `live_rows` rows in use; rows beyond
    are neither read for a result nor zeroed."""
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    T, cap, K, E, N, k = 200, 384, 512, 4, 512, 2
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=55)
    ref = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    (xq, xs), (w1q, w1s), (w2q, w2s) = q["x"], q["w1"], q["w2"]
    xd = torch.zeros(cap, K, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    xd[:T] = xq.to(DEV)
    sd = torch.zeros(cap, K // 32, dtype=torch.uint8, device=DEV).view(torch.float8_e8m0fnu)
    sd[:T] = xs.to(DEV)
    idd = torch.full((cap, k), -1, dtype=torch.int32, device=DEV)
    idd[:T] = ids.to(DEV)
    wd = torch.zeros(cap, k, dtype=torch.float32, device=DEV)
    wd[:T] = wts.to(DEV)
    live = torch.tensor([T], dtype=torch.int32, device=DEV)
    s, e, n = capi.moe_align(idd, E, 128, 1)
    out = torch.full((cap, K), float("nan"), dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_mxfp8(xd, sd, w1q.to(DEV), P.pack_scales_blocked(w1s).to(DEV), w2q.to(DEV),
                         P.pack_scales_blocked(w2s).to(DEV), s, e, n, wd.view(-1), out, k, 128, 64, 4, 4, 1, True,
                         live_rows=live)
    torch.cuda.synchronize()
    assert O.max_rel_to_peak(out[:T].cpu(), ref) <= TOL
    assert torch.isnan(out[T:].float()).all()
    assert capi.device_status() == 0


@pytest.mark.parametrize("stages", [1, 2, 4])
@pytest.mark.parametrize("T,K,E,N,k", [(8, 256, 1, 256, 1), (300, 512, 4, 512, 2), (256, 4096, 8, 512, 4),
                                        (1000, 1024, 16, 768, 8), (700, 256, 3, 1024, 1), (2048, 2048, 32, 2048, 4)])
def test_in_kernel_row_gather(T, K, E, N, k, stages, monkeypatch):
    """Gate/up kernel with the routed rows of x and their scale rows gathered inside the kernel (four LSU warps,
    PMOE_AGATHER=lsu; an option, the pre-pass measured faster) against the row-gather pre-pass (PMOE_AGATHER=pre): the
    same arithmetic per routed row, so both meet the oracle bound and differ from one another only by the order of
    the bf16 reductions into `out`."""
    q, deq, ids, wts = quantised_case(T, K, E, N, k, seed=T + stages)
    ref = O.moe_ref_fp32(deq["x"], deq["w1"], deq["w2"], ids, wts, requant_act=True)
    monkeypatch.setenv("PMOE_AGATHER", "lsu")
    lsu, _ = run_mine(q, ids, wts, True, stages=stages)
    monkeypatch.setenv("PMOE_AGATHER", "pre")
    pre, _ = run_mine(q, ids, wts, True, stages=stages)
    assert torch.isfinite(lsu.float()).all()
    assert O.max_rel_to_peak(lsu, ref) <= TOL
    assert O.max_rel_to_peak(pre, ref) <= TOL
    assert O.max_rel_to_peak(lsu, pre.float()) <= TOL
