"""The benchmarked configurations at (or near) their real sizes, on the kernels and knobs the benchmark uses.

Full-size inputs are generated on the device; the CPU oracle runs on a small slice of the tokens (bounded work:
per token only the weights of the experts it routes to are brought to the host and, for mxfp8, dequantised),
which is valid because every output row depends on its own token alone. Tolerances as everywhere:
2e-2 of the peak against the fp32 oracle (for mxfp8 the requant-aware dequantised fp32 oracle)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


def device_case(T, K, E, N, k, seed, dist="uniform"):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w1 = torch.randn(E, N, K, device=DEV, generator=g, dtype=torch.bfloat16) * K ** -0.5
    w2 = torch.randn(E, K, N // 2, device=DEV, generator=g, dtype=torch.bfloat16) * (N // 2) ** -0.5
    ids, wts = O.make_routing(T, E, k, seed + 1, dist)
    return x, w1, w2, ids, wts


def quantize_on_device(t, chunk=16):
    """The oracle's quantiser (oracle.quantize_mx, plain torch ops) run on the device a few experts at a time."""
    if t.dim() == 2:
        q, s = O.quantize_mx(t)
        return q, s
    qs, ss = [], []
    for i in range(0, t.shape[0], chunk):
        q, s = O.quantize_mx(t[i:i + chunk])
        qs.append(q)
        ss.append(s)
    return torch.cat(qs), torch.cat(ss)


def oracle_rows(tokens, x, w1, w2, ids, wts, scales=None):
    """fp32 oracle rows for `tokens`: per token, its experts' weights only. `scales` = (xs, w1s, w2s) row-major
    e8m0 for mxfp8 operands (then x, w1, w2 are e4m3 and the oracle re-quantises the activation)."""
    rows = []
    for t in tokens:
        e = ids[t].long()
        local = torch.arange(e.numel(), dtype=torch.int32).view(1, -1)
        if scales is None:
            xr, a, b = x[t:t + 1].cpu(), w1[e.to(DEV)].cpu(), w2[e.to(DEV)].cpu()
            rows.append(O.moe_ref_fp32(xr, a, b, local, wts[t:t + 1]))
        else:
            xs, w1s, w2s = scales
            ed = e.to(DEV)
            xr = O.dequantize_mx(x[t:t + 1].cpu(), xs[t:t + 1].cpu())
            a = O.dequantize_mx(w1[ed].cpu(), w1s[ed].cpu())
            b = O.dequantize_mx(w2[ed].cpu(), w2s[ed].cpu())
            rows.append(O.moe_ref_fp32(xr, a, b, local, wts[t:t + 1], requant_act=True))
    return torch.cat(rows)


def run_bf16(x, w1, w2, ids, wts, bpc=1, stages=4, split=True):
    from prime_flash_moe_b200 import capi
    T, K = x.shape
    s, e, n = capi.moe_align(ids.to(DEV), w1.shape[0], 128, bpc)
    out = torch.full((T, K), float("nan"), dtype=torch.bfloat16, device=DEV) if split else \
        torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_bf16(x, w1, w2, s, e, n, wts.to(DEV), out, ids.shape[1], 128, 64, 4, stages, bpc, 1, split)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    return out


def run_mx(xq, xs, w1q, w1p, w2q, w2p, ids, wts, split=True, stages=4):
    from prime_flash_moe_b200 import capi
    T, K = xq.shape
    s, e, n = capi.moe_align(ids.to(DEV), w1q.shape[0], 128, 1)
    out = torch.full((T, K), float("nan"), dtype=torch.bfloat16, device=DEV) if split else \
        torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_mxfp8(xq, xs, w1q, w1p, w2q, w2p, s, e, n, wts.to(DEV), out, ids.shape[1], 128, 64, 4, stages, 1, split)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    return out


def spread(T, n):
    """n token indices spread over the batch (first, last and evenly in between)."""
    return sorted(set([0, T - 1] + [int(i * (T - 1) / max(n - 1, 1)) for i in range(n)]))


def test_c1_mixtral_cta_pairs_full_size(monkeypatch):
    """Configuration 1 exactly as the benchmark runs it: bpc=2 (CTA pairs), stages=4, with the half-empty last
    pairs as single blocks on the one-CTA kernels (default) and as pairs."""
    T, K, E, N, k = 4096, 4096, 8, 28672, 2
    x, w1, w2, ids, wts = device_case(T, K, E, N, k, seed=7)
    toks = spread(T, 16)
    ref = oracle_rows(toks, x, w1, w2, ids, wts)
    one = run_bf16(x, w1, w2, ids, wts, bpc=1)
    assert O.max_rel_to_peak(one[toks].cpu(), ref) <= TOL
    for tails in ("1", "0"):
        monkeypatch.setenv("PMOE_PAIR_TAILS", tails)
        out = run_bf16(x, w1, w2, ids, wts, bpc=2)
        assert torch.isfinite(out.float()).all()
        assert O.max_rel_to_peak(out.cpu(), one.cpu().float()) <= TOL
        assert O.max_rel_to_peak(out[toks].cpu(), ref) <= TOL


@pytest.mark.parametrize("T", [8192, 16384])
def test_c2_qwen3_bf16_default_paths(T):
    """Configuration 2 at T=8192 (in-kernel row gather, one row block per tile) and T=16384 (two row blocks per
    tile: 1024 routed rows per expert), whatever the launcher picks by default."""
    K, E, N, k = 2048, 128, 1536, 8
    x, w1, w2, ids, wts = device_case(T, K, E, N, k, seed=T)
    out = run_bf16(x, w1, w2, ids, wts)
    assert torch.isfinite(out.float()).all()
    toks = spread(T, 32)
    assert O.max_rel_to_peak(out[toks].cpu(), oracle_rows(toks, x, w1, w2, ids, wts)) <= TOL


def test_c2_qwen3_mxfp8_T8192():
    T, K, E, N, k = 8192, 2048, 128, 1536, 8
    x, w1, w2, ids, wts = device_case(T, K, E, N, k, seed=5)
    import prime_flash_moe_b200 as P
    (xq, xs), (w1q, w1s), (w2q, w2s) = quantize_on_device(x), quantize_on_device(w1), quantize_on_device(w2)
    del w1, w2
    out = run_mx(xq, xs, w1q, P.pack_scales_blocked(w1s), w2q, P.pack_scales_blocked(w2s), ids, wts)
    assert torch.isfinite(out.float()).all()
    toks = spread(T, 24)
    ref = oracle_rows(toks, xq, w1q, w2q, ids, wts, scales=(xs, w1s, w2s))
    assert O.max_rel_to_peak(out[toks].cpu(), ref) <= TOL


def test_c3_deepseek_shape_mxfp8():
    """Configuration 3's layer (K=7168, E=256, N=4096, top_k=8) on 2048 tokens, both pipelines."""
    import prime_flash_moe_b200 as P
    T, K, E, N, k = 2048, 7168, 256, 4096, 8
    g = torch.Generator(device=DEV).manual_seed(33)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w1q, w1s, w2q, w2s = [], [], [], []
    for _ in range(0, E, 32):            # 32 experts at a time: the bf16 originals never exist all at once
        a = torch.randn(32, N, K, device=DEV, generator=g, dtype=torch.bfloat16) * K ** -0.5
        b = torch.randn(32, K, N // 2, device=DEV, generator=g, dtype=torch.bfloat16) * (N // 2) ** -0.5
        q, s = quantize_on_device(a)
        w1q.append(q), w1s.append(s)
        q, s = quantize_on_device(b)
        w2q.append(q), w2s.append(s)
        del a, b
    w1q, w1s, w2q, w2s = torch.cat(w1q), torch.cat(w1s), torch.cat(w2q), torch.cat(w2s)
    ids, wts = O.make_routing(T, E, k, 34)
    xq, xs = quantize_on_device(x)
    toks = spread(T, 8)
    ref = oracle_rows(toks, xq, w1q, w2q, ids, wts, scales=(xs, w1s, w2s))
    w1p, w2p = P.pack_scales_blocked(w1s), P.pack_scales_blocked(w2s)
    for split in (True, False):
        out = run_mx(xq, xs, w1q, w1p, w2q, w2p, ids, wts, split=split)
        assert torch.isfinite(out.float()).all()
        assert O.max_rel_to_peak(out[toks].cpu(), ref) <= TOL


@pytest.mark.parametrize("dtype", ["bf16", "mxfp8"])
def test_c4_zipf_shape(dtype):
    """Configuration 4's layer (K=4096, E=128, N=3072, top_k=8) with Zipf routing on 8192 tokens: empty experts,
    -1 padding rows, a few experts with thousands of rows."""
    import prime_flash_moe_b200 as P
    T, K, E, N, k = 8192, 4096, 128, 3072, 8
    x, w1, w2, _, wts = device_case(T, K, E, N, k, seed=44, dist="zipf")
    # Zipf over 120 of the 128 experts, placed by a seeded permutation: eight experts receive nothing
    ids120, _ = O.make_routing(T, 120, k, 45, "zipf")
    place = torch.randperm(E, generator=torch.Generator().manual_seed(46))[:120].to(torch.int32)
    ids = place[ids120.long()].contiguous()
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E)
    assert int((counts == 0).sum()) == 8 and int(counts.max()) > 2048, "the case must hold empty and hot experts"
    toks = spread(T, 24)
    if dtype == "bf16":
        out = run_bf16(x, w1, w2, ids, wts)
        ref = oracle_rows(toks, x, w1, w2, ids, wts)
    else:
        (xq, xs), (w1q, w1s), (w2q, w2s) = quantize_on_device(x), quantize_on_device(w1), quantize_on_device(w2)
        del w1, w2
        out = run_mx(xq, xs, w1q, P.pack_scales_blocked(w1s), w2q, P.pack_scales_blocked(w2s), ids, wts)
        ref = oracle_rows(toks, xq, w1q, w2q, ids, wts, scales=(xs, w1s, w2s))
    assert torch.isfinite(out.float()).all()
    assert O.max_rel_to_peak(out[toks].cpu(), ref) <= TOL


def backward_rows_oracle(tokens, x, w1, w2, ids, wts, d_out):
    """Autograd-through-the-fp32-oracle gradients d_x[t], d_topk_weights[t] for `tokens` (each depends on its own
    token and the weights of the experts it routes to only)."""
    dx, dwt = [], []
    for t in tokens:
        e = ids[t].long()
        local = torch.arange(e.numel(), dtype=torch.int32).view(1, -1)
        g = O.moe_backward_ref_fp32(x[t:t + 1].cpu(), w1[e.to(DEV)].cpu(), w2[e.to(DEV)].cpu(), local, wts[t:t + 1],
                                    d_out[t:t + 1].cpu())
        dx.append(g[0])
        dwt.append(g[3])
    return torch.cat(dx), torch.cat(dwt)


@pytest.mark.parametrize("name,T,K,E,N,k,kept", [
    ("c1", 4096, 4096, 8, 28672, 2, False),        # weight gradients on CTA pairs, pre-activations recomputed
    ("c1", 4096, 4096, 8, 28672, 2, True),         # ... kept by the forward call
    ("c1", 4096, 4096, 8, 28672, 2, 2),            # ... kept by the CTA-pair forward (routing tables padded to 256 rows)
    ("c2", 8192, 2048, 128, 1536, 8, False),
])
def test_backward_full_size(name, T, K, E, N, k, kept):
    """The backward pass on benchmark layers at full size: d_x and d_topk_weights of sampled tokens against autograd
    through the fp32 oracle, weight gradients of sampled experts on a slice of 256 hidden columns against the
    slice-wise restatement (oracle.moe_backward_expert_slice_ref), linearity in d_out over the whole tensors."""
    from prime_flash_moe_b200 import capi
    H = N // 2
    x, w1, w2, ids, wts = device_case(T, K, E, N, k, seed=41)
    d_out = torch.randn(T, K, device=DEV, generator=torch.Generator(device=DEV).manual_seed(42)).to(torch.bfloat16)
    bpc = 2 if kept == 2 else 1
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, bpc)
    dwts = wts.to(DEV)
    gate_up = None
    if kept:
        _, gate_up = capi.fused_moe_bf16_keep(x, w1, w2, s, e, n, dwts, torch.empty_like(x), k, bpc=bpc)
    d_x, d_w1, d_w2, d_wt = capi.fused_moe_bf16_backward(x, w1, w2, d_out, s, e, n, dwts, k, gate_up=gate_up)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for g in (d_x, d_w1, d_w2, d_wt):
        assert torch.isfinite(g.float()).all()
    toks = spread(T, 12)
    ref_dx, ref_dwt = backward_rows_oracle(toks, x, w1, w2, ids, wts, d_out)
    assert O.max_rel_to_peak(d_x[toks].cpu(), ref_dx) <= TOL
    assert O.max_rel_to_peak(d_wt[toks].cpu(), ref_dwt) <= TOL
    for ex, h0 in ((0, 0), (E - 1, H - 256)):
        tok, route = torch.nonzero(ids == ex, as_tuple=True)
        hs = slice(h0, h0 + 256)
        want = O.moe_backward_expert_slice_ref(x[tok.to(DEV)].cpu(), d_out[tok.to(DEV)].cpu(), wts[tok, route],
                                               w1[ex, hs].cpu(), w1[ex, H + h0:H + h0 + 256].cpu(), w2[ex][:, hs].cpu())
        got = (d_w1[ex, hs], d_w1[ex, H + h0:H + h0 + 256], d_w2[ex][:, hs])
        for g, w in zip(got, want):
            assert O.max_rel_to_peak(g.cpu(), w) <= TOL
    # linearity: doubling d_out doubles every gradient (exact in bf16 up to the order of the fp32 atomics of d_wt)
    twice = capi.fused_moe_bf16_backward(x, w1, w2, (d_out.float() * 2).to(torch.bfloat16), s, e, n, dwts, k,
                                         gate_up=gate_up)
    torch.cuda.synchronize()
    for g, g2 in zip((d_x, d_w1, d_w2), twice[:3]):
        assert torch.equal((g.float() * 2).to(torch.bfloat16), g2)
    assert O.max_rel_to_peak(twice[3].cpu(), d_wt.cpu() * 2) <= 1e-5
