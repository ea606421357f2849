"""fused_moe_bf16 on the GPU against the CPU oracle (fp32 and the reference's bf16 test oracle), the
golden vectors, and the reference's own kernels when oracle/_ref is built.

Tolerance (stated by the task): max|out - ref| <= 2e-2 * max|ref| against the all-fp32 oracle; plus the
reference's own gates rel_clamp_10 <= 0.02, rel_clamp_1 <= 0.10 (test/test.py:9-10) on its own input
distribution."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O, ref_kernels as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


def run_mine(x, w1, w2, ids, wts, split, stages=4, bn=64, wn=4, via="capi", bpc=1):
    from prime_flash_moe_b200 import capi
    import prime_flash_moe_b200 as P
    E = w1.shape[0]
    T, K = x.shape
    k = ids.shape[1]
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, bpc)
    out = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV) if not split else \
        torch.full((T, K), float("nan"), dtype=torch.bfloat16, device=DEV)   # split=True must overwrite
    args = (x.to(DEV), w1.to(DEV), w2.to(DEV), s, e, n, wts.to(DEV), out, k, 128, bn, wn, stages, bpc, 1, split)
    if via == "capi":
        capi.fused_moe_bf16(*args)
    else:
        ret = P.fused_moe_bf16(*args)
        assert ret is out
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    return out.cpu()


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("T,K,E,N,k", [
    (1, 128, 2, 256, 1), (8, 128, 1, 256, 1), (64, 512, 4, 512, 2), (130, 256, 5, 768, 3),
    (256, 4096, 8, 512, 4),      # benchmark configuration 0
    (300, 1024, 8, 1024, 4), (1000, 384, 16, 256, 8),
])
def test_vs_fp32_oracle(T, K, E, N, k, split):
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=T + K)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    out = run_mine(x, w1, w2, ids, wts, split)
    assert torch.isfinite(out.float()).all()
    assert O.max_rel_to_peak(out, ref) <= TOL


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("bn,wn", [(64, 4), (32, 8)])
@pytest.mark.parametrize("stages", [1, 2, 3, 4, 5])
def test_knobs(split, bn, wn, stages):
    if split and stages == 5:
        pytest.skip("split=True accepts stages <= 4 (checked in test_argument_checks)")
    x, w1, w2, ids, wts = O.make_case(200, 512, 6, 512, 3, seed=stages)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    out = run_mine(x, w1, w2, ids, wts, split, stages=stages, bn=bn, wn=wn, via="torch")
    assert O.max_rel_to_peak(out, ref) <= TOL


@pytest.mark.parametrize("tails", ["1", "0"])
@pytest.mark.parametrize("bn,wn,stages", [(64, 4, 1), (64, 4, 4), (32, 8, 3)])
@pytest.mark.parametrize("T,K,E,N,k", [(8, 128, 1, 256, 1), (300, 512, 4, 512, 2), (256, 4096, 8, 512, 4),
                                        (1000, 1024, 16, 768, 8), (700, 256, 3, 1024, 1)])
def test_two_cta_pipeline(T, K, E, N, k, bn, wn, stages, tails, monkeypatch):
    """bpc = 2: CTA pairs with cta_group::2 MMAs on routing tables padded to 256 rows per expert; by default the
    half-empty last pair of an expert runs as a single block on the one-CTA kernels (PMOE_PAIR_TAILS)."""
    monkeypatch.setenv("PMOE_PAIR_TAILS", tails)
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=T + stages)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    out = run_mine(x, w1, w2, ids, wts, True, stages=stages, bn=bn, wn=wn, bpc=2)
    assert torch.isfinite(out.float()).all()
    assert O.max_rel_to_peak(out, ref) <= TOL
    # same arithmetic as the one-CTA pipeline: only the order of the top_k bf16 reductions into `out`
    # differs (each is within TOL of the oracle; with top_k = 8 the two orders differ by up to ~1.3e-2)
    one = run_mine(x, w1, w2, ids, wts, True, stages=stages, bn=bn, wn=wn, bpc=1)
    assert O.max_rel_to_peak(out, one) <= TOL


def test_golden_vectors(golden):
    """Outputs of the reference's moe_naive_from_topk (test/test.py:13-48) stored in tests/golden."""
    for case in golden["moe_bf16"]:
        for split in (True, False):
            out = run_mine(case["x"], case["w1"], case["w2"], case["topk_ids"], case["topk_weights"], split)
            assert O.max_rel_to_peak(out, case["out"]) <= TOL


@pytest.mark.parametrize("T", [8, 32, 128, 256])
@pytest.mark.parametrize("E,N,K", [(8, 256, 4096), (37, 512, 4096), (257, 256, 7168), (8, 512, 7168)])
def test_reference_sweep_distribution(T, E, N, K):
    """Inputs, routing and gates of the reference's bf16 sweep (test/test.py:133-191): x ~ N(0, 0.05^2),
    weights 0.05*N(0,1), top_k = 9 with duplicates allowed and the last expert forced, split=False,
    config (128, 32, 8, stages=1); gates rel_clamp_10 <= 0.02 and rel_clamp_1 <= 0.10."""
    g = torch.Generator().manual_seed(T * 1000 + E)
    x = (torch.randn(T, K, generator=g) * 0.05).to(torch.bfloat16)
    w1 = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, K, N // 2, generator=g) * 0.05).to(torch.bfloat16)
    ids = torch.randint(0, E - 1, (T, 9), generator=g, dtype=torch.int32)
    ids[:, -1] = E - 1
    wts = torch.softmax(torch.randn(T, 9, generator=g), dim=-1)
    ref = O.moe_ref_bf16(x, w1, w2, ids, wts)
    for split in (False, True):
        out = run_mine(x, w1, w2, ids, wts, split, stages=1, bn=32, wn=8)
        assert torch.isfinite(out.float()).all()
        assert O.rel_clamp(out, ref, 10.0) <= 0.02
        assert O.rel_clamp(out, ref, 1.0) <= 0.10
        assert O.max_rel_to_peak(out, O.moe_ref_fp32(x, w1, w2, ids, wts)) <= TOL


def test_padding_and_empty_experts():
    """Zipf routing over many experts: most experts empty, -1 padding rows inside blocks."""
    x, w1, w2, ids, wts = O.make_case(96, 256, 64, 256, 4, seed=9, dist="zipf")
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    for split in (True, False):
        assert O.max_rel_to_peak(run_mine(x, w1, w2, ids, wts, split), ref) <= TOL


def test_split_false_accumulates_and_split_true_overwrites():
    from prime_flash_moe_b200 import capi
    x, w1, w2, ids, wts = O.make_case(64, 256, 4, 256, 2, seed=4)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    s, e, n = capi.moe_align(ids.to(DEV), 4, 128, 1)
    args = (x.to(DEV), w1.to(DEV), w2.to(DEV), s, e, n, wts.to(DEV))
    out = torch.ones(64, 256, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_bf16(*args, out, 2, split=False)
    assert O.max_rel_to_peak(out.cpu().float() - 1.0, ref) <= 3e-2       # accumulated on top of the ones
    capi.fused_moe_bf16(*args, out, 2, split=True)
    assert O.max_rel_to_peak(out.cpu(), ref) <= TOL                       # zeroed by the library


def test_argument_checks():
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    x, w1, w2, ids, wts = O.make_case(16, 256, 2, 256, 2, seed=1)
    s, e, n = capi.moe_align(ids.to(DEV), 2, 128, 1)
    out = torch.zeros(16, 256, dtype=torch.bfloat16, device=DEV)
    a = [x.to(DEV), w1.to(DEV), w2.to(DEV), s, e, n, wts.to(DEV), out, 2, 128, 64, 4, 2, 1, 1, True]

    def bad(i, v):
        b = list(a)
        b[i] = v
        with pytest.raises(RuntimeError):
            P.fused_moe_bf16(*b)

    bad(9, 64)            # block_m
    bad(10, 16)           # block_n / warp_n pair
    bad(12, 6)            # stages
    bad(12, 5)            # stages 5 with split=True
    bad(14, 2)            # cpc
    bad(13, 3)            # bpc must be 1 or 2
    b2 = list(a); b2[13] = 2; b2[15] = False
    with pytest.raises(RuntimeError):
        P.fused_moe_bf16(*b2)          # bpc=2 needs split=True
    bad(0, x.to(DEV).float())          # dtype
    bad(0, x.to(DEV)[:, ::2])          # contiguity / K mismatch
    bad(6, wts.to(DEV).double())       # topk_weights dtype
    assert capi.device_status() == 0


def test_full_size_properties_mixtral():
    """Benchmark configuration 1 (Mixtral-8x7B layer, T=4096) at full size, checked through properties
    that need no CPU reference: the two pipelines agree with each other, rows of tokens are independent
    of the rest of the batch (a 64-token slice reproduces the same rows), and every row is finite."""
    T, K, E, N, k = 4096, 4096, 8, 28672, 2
    g = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, N, K, device=DEV, generator=g, dtype=torch.bfloat16) * K ** -0.5)
    w2 = (torch.randn(E, K, N // 2, device=DEV, generator=g, dtype=torch.bfloat16) * (N // 2) ** -0.5)
    ids, wts = O.make_routing(T, E, k, seed=8)
    a = run_mine(x, w1, w2, ids, wts, True)
    assert torch.isfinite(a.float()).all()
    sub = run_mine(x[:64], w1, w2, ids[:64], wts[:64], True)
    # same arithmetic per routed row; the bf16 reductions into an output element land in a different order
    assert O.max_rel_to_peak(sub, a[:64]) <= TOL
    # CPU oracle on the same 64 tokens (bounded work: 64 tokens x 2 experts each)
    ref = O.moe_ref_fp32(x[:64].cpu(), w1.cpu(), w2.cpu(), ids[:64], wts[:64])
    assert O.max_rel_to_peak(a[:64], ref) <= TOL
    # The single-GEMM-launch pipeline reduces its top_k * H/128 = 224 split-K partials per element in
    # fp32, so it meets the same gate (the reference's bf16 atomics do not at this H).
    b = run_mine(x, w1, w2, ids, wts, False)
    assert torch.isfinite(b.float()).all()
    assert O.max_rel_to_peak(b, a) <= TOL
    assert O.max_rel_to_peak(b[:64], ref) <= TOL


@pytest.mark.skipif(not R.available(), reason="oracle/_ref (reference kernels) not built")
@pytest.mark.parametrize("T,K,E,N,k", [(256, 4096, 8, 512, 4), (128, 2048, 128, 1536, 8), (2048, 2048, 32, 2048, 4)])
def test_vs_reference_kernels(T, K, E, N, k):
    """Same seeded inputs through the reference's own sm_100a kernels (both of its pipelines)."""
    from prime_flash_moe_b200 import capi
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=T)
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, 1)
    xd, w1d, w2d, wd = x.to(DEV), w1.to(DEV), w2.to(DEV), wts.to(DEV)
    ref32 = O.moe_ref_fp32(x, w1, w2, ids, wts)
    for split in (False, True):
        ref_out = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
        R.fused_moe_bf16(xd, w1d, w2d, s, e, n, wd, ref_out, k, 128, 64, 4, 2, 1, 1, split)
        torch.cuda.synchronize()
        mine = run_mine(x, w1, w2, ids, wts, split)
        # the reference's own result sits up to ~1.9e-2 from the fp32 oracle on these shapes (bf16
        # atomics over top_k * H/128 partials), so two correct implementations may differ by more than
        # one tolerance: bound the distance by two tolerances, and hold this library to the gate itself
        # (the reference's bf16 atomics make its own result vary from run to run; observed distance to
        # this library 0.6e-2 .. 2.4e-2, so the bound is two tolerances to keep the check stable)
        assert O.max_rel_to_peak(mine, ref_out.cpu()) <= 2.0 * TOL
        assert O.max_rel_to_peak(mine, ref32) <= TOL


@pytest.mark.parametrize("split", [True, False])
def test_cuda_graph_capture_and_replay(split):
    """The operators enqueue on the caller's stream without synchronising the host, so a CUDA graph can
    capture them (the reference's benchmark times graph replays, benchmark/benchmark.py:355-370)."""
    import prime_flash_moe_b200 as P
    x, w1, w2, ids, wts = O.make_case(96, 512, 8, 512, 2, seed=21)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    xd, w1d, w2d, idd, wd = x.to(DEV), w1.to(DEV), w2.to(DEV), ids.to(DEV), wts.to(DEV)
    out = torch.zeros(96, 512, dtype=torch.bfloat16, device=DEV)

    def step():
        s, e, n = torch.ops.prime_moe.moe_align(idd, 8, 128, 1)
        if not split:
            out.zero_()
        P.fused_moe_bf16(xd, w1d, w2d, s, e, n, wd, out, 2, 128, 64, 4, 4, 1, 1, split)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()                      # warm-up outside the capture (lazy initialisation)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert O.max_rel_to_peak(out.cpu(), ref) <= TOL


FEW_ROW_CASES = [
    (1, 128, 2, 256, 1), (1, 2048, 128, 1536, 8), (16, 2048, 128, 1536, 8),   # decode shapes of the Qwen3 layer
    (8, 256, 1, 512, 1),
    (32, 128, 1, 256, 1),     # exactly 32 routed rows in the block: the largest short block
    (33, 128, 1, 256, 1),     # 33 rows: a full block again
    (8, 7168, 4, 512, 4),     # long rows (DeepSeek-V3 hidden size)
    (5, 384, 7, 768, 3),      # K a multiple of 128 only, H = 384
    (200, 512, 6, 512, 3),    # short and full blocks mixed
]


@pytest.mark.parametrize("agather", ["auto", "tma4"])
@pytest.mark.parametrize("T,K,E,N,k", FEW_ROW_CASES)
def test_short_row_blocks(T, K, E, N, k, agather, monkeypatch):
    """Row blocks holding at most 32 routed rows load and store only those rows of the A operand and of the
    activation tile (short TMA boxes); PMOE_SHORT_A=0 moves whole 128-row tiles. Both must meet the oracle bound,
    and they run the same arithmetic on the routed rows, so their outputs must be identical up to the order of
    the bf16 reductions into `out`."""
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=3 * T + K)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    if agather != "auto":       # auto = row-gather pre-pass for calls this small
        monkeypatch.setenv("PMOE_AGATHER", agather)
    monkeypatch.setenv("PMOE_SHORT_A", "3")
    short = run_mine(x, w1, w2, ids, wts, True)
    monkeypatch.setenv("PMOE_SHORT_A", "0")
    full = run_mine(x, w1, w2, ids, wts, True)
    assert torch.isfinite(short.float()).all()
    assert O.max_rel_to_peak(short, ref) <= TOL
    assert O.max_rel_to_peak(full, ref) <= TOL
    # same arithmetic per routed row; the top_k bf16 reductions into an output element land in a different order
    # from run to run (with top_k = 8 two orders differ by up to ~1.3e-2 of the peak)
    assert O.max_rel_to_peak(short, full.float()) <= TOL


@pytest.mark.parametrize("agather", ["pre", "lsu"])
@pytest.mark.parametrize("bn,wn,stages", [(64, 4, 1), (64, 4, 4), (32, 8, 2)])
@pytest.mark.parametrize("T,K,E,N,k", [(8, 128, 1, 256, 1), (300, 512, 4, 512, 2), (256, 4096, 8, 512, 4),
                                        (1000, 1024, 16, 768, 8), (700, 256, 3, 1024, 1), (2048, 2048, 32, 2048, 4)])
def test_dual_block_tiles(T, K, E, N, k, bn, wn, stages, agather, monkeypatch):
    """Gate/up kernel with two row blocks per tile (consecutive blocks of one expert share the weight slots;
    blocks of different experts and an odd last block run as single passes) against one block per tile: the
    same arithmetic per routed row, so the outputs differ only by the order of the bf16 reductions."""
    monkeypatch.setenv("PMOE_AGATHER", agather)
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=T + stages)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    monkeypatch.setenv("PMOE_DUAL", "1")
    dual = run_mine(x, w1, w2, ids, wts, True, stages=stages, bn=bn, wn=wn)
    monkeypatch.setenv("PMOE_DUAL", "0")
    one = run_mine(x, w1, w2, ids, wts, True, stages=stages, bn=bn, wn=wn)
    assert torch.isfinite(dual.float()).all()
    assert O.max_rel_to_peak(dual, ref) <= TOL
    assert O.max_rel_to_peak(one, ref) <= TOL
    assert O.max_rel_to_peak(dual, one.float()) <= TOL


@pytest.mark.parametrize("bpc", [1, 2])
def test_ex_entry_point_live_rows_and_output_addresses(bpc):
    """`pmoe_fused_moe_bf16_ex` (the expert-parallel mode's entry point). live_rows: buffers sized for a worst case,
    only the leading rows in use - the library zeroes just those rows of `out`. out_rows: every output row has its
    own address (here rows of a second buffer in permuted order; across GPUs: rows of the source rank's buffer) and
    the down kernels ADD their results there, zeroing nothing."""
    from prime_flash_moe_b200 import capi
    T, cap, K, E, N, k = 300, 512, 512, 4, 512, 2
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=77)
    ref = O.moe_ref_fp32(x, w1, w2, ids, wts)
    xd = torch.full((cap, K), float("nan"), dtype=torch.bfloat16, device=DEV)      # rows beyond T are never read
    xd[:T] = x.to(DEV)
    idd = torch.full((cap, k), -1, dtype=torch.int32, device=DEV)
    idd[:T] = ids.to(DEV)
    wd = torch.zeros(cap, k, dtype=torch.float32, device=DEV)
    wd[:T] = wts.to(DEV)
    live = torch.tensor([T], dtype=torch.int32, device=DEV)
    s, e, n = capi.moe_align(idd, E, 128, bpc)
    out = torch.full((cap, K), float("nan"), dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_bf16(xd, w1.to(DEV), w2.to(DEV), s, e, n, wd.view(-1), out, k, 128, 64, 4, 4, bpc, 1, True, live_rows=live)
    torch.cuda.synchronize()
    assert O.max_rel_to_peak(out[:T].cpu(), ref) <= TOL
    assert torch.isnan(out[T:].float()).all(), "rows beyond live_rows must be left alone"
    # every output row at its own address: row i of the result lands in row perm[i] of `y`
    perm = torch.randperm(cap, generator=torch.Generator().manual_seed(3))
    y = torch.zeros(cap, K, dtype=torch.bfloat16, device=DEV)
    table = (y.data_ptr() + perm.to(torch.int64) * K * 2).to(DEV)
    out.fill_(float("nan"))
    capi.fused_moe_bf16(xd, w1.to(DEV), w2.to(DEV), s, e, n, wd.view(-1), out, k, 128, 64, 4, 4, bpc, 1, True, live_rows=live,
                        out_rows=table)
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all(), "`out` itself is not written when out_rows is given"
    assert O.max_rel_to_peak(y[perm[:T].to(DEV)].cpu(), ref) <= TOL
    assert float(y[perm[T:].to(DEV)].float().abs().max()) == 0.0
    assert capi.device_status() == 0
    with pytest.raises(RuntimeError):      # a split=False call cannot address rows individually
        capi.fused_moe_bf16(xd, w1.to(DEV), w2.to(DEV), s, e, n, wd.view(-1), out, k, 128, 64, 4, 4, 1, 1, False,
                            out_rows=table)
