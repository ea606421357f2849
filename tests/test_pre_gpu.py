"""The two steps ahead of the fused MoE FFN on the GPU: the MX activation quantiser against the CPU oracle and
the golden vectors made by executing the reference's quantiser (bit-exact), and the router against
torch.softmax + torch.topk (ids exact, weights <= 1e-6, ties to the lower expert index)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _u8(t):
    return t.view(torch.uint8).cpu()


@pytest.mark.parametrize("T,K", [(1, 32), (3, 96), (257, 2048), (64, 7168), (1000, 4096)])
@pytest.mark.parametrize("via", ["capi", "torch"])
def test_quantize_mx_bit_exact(T, K, via):
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    g = torch.Generator().manual_seed(T + K)
    x = torch.randn(T, K, generator=g)
    x[0, :32] = 0.0                                     # an all-zero block: exponent clamps at 0
    x[-1, -32:] *= 1e-30                                # tiny block
    x[T // 2, :32] *= 3e4                               # large block
    if T > 2:
        x[1, 5] = 6e4                                   # one outlier saturating its neighbours' resolution
    x = x.to(torch.bfloat16)
    q_ref, s_ref = O.quantize_mx(x)
    q, s = (capi.quantize_mx if via == "capi" else P.quantize_mx)(x.to(DEV))
    torch.cuda.synchronize()
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float8_e8m0fnu
    assert torch.equal(_u8(s), s_ref.view(torch.uint8))
    assert torch.equal(_u8(q), q_ref.view(torch.uint8))


def test_quantize_mx_golden(golden):
    """Inputs and outputs of the reference's own quantiser (test/test_mxfp8.py:21-38), stored in tests/golden."""
    from prime_flash_moe_b200 import capi
    used = 0
    for case in golden["quant"]:
        x = case["input"]
        xb = x.to(torch.bfloat16)
        if not torch.equal(xb.to(x.dtype), x):
            continue                                    # not representable in bf16: outside this entry point's domain
        q, s = capi.quantize_mx(xb.contiguous().to(DEV))
        torch.cuda.synchronize()
        assert torch.equal(_u8(q), case["q"])
        assert torch.equal(_u8(s), case["scales"])
        used += 1
    assert used >= 1


def test_quantize_mx_with_row_gather():
    """row_index: output row r = quantised x[row_index[r]] (the expert-parallel dispatch gather fused in);
    an index outside x gives a row of zeros with zero exponents."""
    from prime_flash_moe_b200 import capi
    g = torch.Generator().manual_seed(5)
    x = torch.randn(500, 1024, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 500, (1300,), generator=g, dtype=torch.int32)
    idx[17] = -1
    idx[18] = 500
    q, s = capi.quantize_mx(x.to(DEV), idx.to(DEV))
    torch.cuda.synchronize()
    safe = idx.clamp(0, 499).long()
    q_ref, s_ref = O.quantize_mx(x[safe])
    q_ref, s_ref = q_ref.view(torch.uint8).clone(), s_ref.view(torch.uint8).clone()
    q_ref[17:19] = 0
    s_ref[17:19] = 0
    assert torch.equal(_u8(q), q_ref) and torch.equal(_u8(s), s_ref)


def test_quantised_activations_feed_the_fused_op():
    """bf16 activations -> pmoe_quantize_mx -> fused_moe_mxfp8 equals the path with the oracle's quantiser."""
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    T, K, E, N, k = 200, 512, 8, 512, 2
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=12)
    (w1q, w1s), (w2q, w2s) = O.quantize_mx(w1), O.quantize_mx(w2)
    xq, xs = capi.quantize_mx(x.to(DEV))
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, 1)
    out = torch.empty(T, K, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_mxfp8(xq, xs, w1q.to(DEV), P.pack_scales_blocked(w1s).to(DEV), w2q.to(DEV),
                         P.pack_scales_blocked(w2s).to(DEV), s, e, n, wts.to(DEV), out, k)
    torch.cuda.synchronize()
    xq_o, xs_o = O.quantize_mx(x)
    ref = O.moe_ref_fp32(O.dequantize_mx(xq_o, xs_o), O.dequantize_mx(w1q, w1s), O.dequantize_mx(w2q, w2s), ids, wts,
                         requant_act=True)
    assert O.max_rel_to_peak(out.cpu(), ref) <= 2e-2
    assert capi.device_status() == 0


@pytest.mark.parametrize("renorm", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (300, 8, 2), (1000, 128, 8), (513, 256, 8), (77, 100, 5), (64, 1024, 32),
                                   (9, 33, 33 - 1)])
def test_route_topk_matches_torch(T, E, k, dtype, renorm):
    from prime_flash_moe_b200 import capi
    g = torch.Generator().manual_seed(T * 7 + E)
    if dtype == torch.bfloat16:
        # distinct bf16 values per row so that the selection is unique: E consecutive bf16 bit patterns
        # (values from 2^-7 upwards), randomly permuted per row
        base = (0x3C00 + torch.arange(E, dtype=torch.int32)).to(torch.int16).view(torch.bfloat16)
        logits = torch.stack([base[torch.randperm(E, generator=g)] for _ in range(T)])
    else:
        logits = torch.randn(T, E, generator=g)
    ids, wts = capi.route_topk(logits.to(DEV), k, renorm)
    torch.cuda.synchronize()
    lf = logits.float()
    top_v, top_i = torch.topk(lf, k, dim=-1)
    ref_w = torch.softmax(top_v, dim=-1) if renorm else torch.softmax(lf, dim=-1).gather(1, top_i)
    assert torch.equal(ids.cpu().long(), top_i)
    assert (wts.cpu() - ref_w).abs().max().item() <= 1e-6
    if renorm:
        assert (wts.cpu().sum(-1) - 1).abs().max().item() <= 1e-5


def test_route_topk_tie_rule_and_torch_op():
    """Equal logits go to the lower expert index; the torch operator returns the same as the C ABI."""
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    logits = torch.zeros(4, 64)
    logits[1, 40] = 1.0
    logits[2, [5, 50]] = 2.0
    logits[3] = torch.arange(64).flip(0).float()
    ids, wts = P.route_topk(logits.to(DEV), 4)
    ids2, wts2 = capi.route_topk(logits.to(DEV), 4)
    torch.cuda.synchronize()
    assert ids.cpu().tolist() == [[0, 1, 2, 3], [40, 0, 1, 2], [5, 50, 0, 1], [0, 1, 2, 3]]
    assert torch.equal(ids, ids2) and torch.equal(wts, wts2)
    assert torch.allclose(wts[0].cpu(), torch.full((4,), 0.25))


def test_route_then_align_then_moe():
    """logits -> route_topk -> moe_align -> fused_moe_bf16 with no host round trip equals the oracle fed with
    torch's routing of the same logits."""
    from prime_flash_moe_b200 import capi
    T, K, E, N, k = 256, 512, 16, 512, 4
    x, w1, w2, _, _ = O.make_case(T, K, E, N, k, seed=31)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(32))
    ids, wts = capi.route_topk(logits.to(DEV), k)
    s, e, n = capi.moe_align(ids, E, 128, 1)
    out = torch.empty(T, K, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_bf16(x.to(DEV), w1.to(DEV), w2.to(DEV), s, e, n, wts, out, k)
    torch.cuda.synchronize()
    tv, ti = torch.topk(logits, k, dim=-1)
    ref = O.moe_ref_fp32(x, w1, w2, ti.to(torch.int32), torch.softmax(tv, -1))
    assert O.max_rel_to_peak(out.cpu(), ref) <= 2e-2


@pytest.mark.parametrize("via", ["capi", "torch"])
@pytest.mark.parametrize("T,E,k,bpc,dtype", [
    (64, 8, 2, 1, torch.float32),            # one CTA aligns it: router kernel + small align kernel
    (4096, 8, 2, 2, torch.float32),          # n = 8192, E <= 256: still one CTA
    (8192, 128, 8, 1, torch.float32),        # fused router + histogram kernel, then the scatter pass
    (16384, 256, 8, 1, torch.bfloat16),
    (20000, 64, 4, 2, torch.float32),
    (9000, 100, 5, 1, torch.float32),        # top_k = 5 does not divide a CTA's id range: the separate kernels
    (3000, 1024, 8, 1, torch.float32),
])
def test_route_topk_align_equals_the_two_separate_calls(T, E, k, bpc, dtype, via):
    """Router fused with the moe_align histogram pass: all five outputs identical, bit for bit, to route_topk
    followed by moe_align on its ids - and the routing tables to the CPU restatement of the reference's."""
    import numpy as np
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    g = torch.Generator().manual_seed(T + E)
    if dtype == torch.bfloat16:
        base = (0x3C00 + torch.arange(E, dtype=torch.int32)).to(torch.int16).view(torch.bfloat16)
        logits = torch.stack([base[torch.randperm(E, generator=g)] for _ in range(T)])
    else:
        logits = torch.randn(T, E, generator=g)
    ld = logits.to(DEV)
    if via == "capi":
        ids, wts, s, e, n = capi.route_topk_align(ld, k, True, 128, bpc)
    else:
        ids, wts, s, e, n = P.route_topk_align(ld, k, True, 128, bpc)
    ids2, wts2 = capi.route_topk(ld, k, True)
    s2, e2, n2 = capi.moe_align(ids2, E, 128, bpc)
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2) and torch.equal(wts, wts2)
    assert torch.equal(s, s2) and torch.equal(e, e2) and torch.equal(n, n2)
    want = O.moe_align_spec(ids.cpu().numpy(), E, 128, bpc)
    for got, ref in zip((s, e, n), want):
        assert np.array_equal(got.cpu().numpy(), ref)
    assert capi.device_status() == 0


def test_argument_checks():
    from prime_flash_moe_b200 import capi
    lib = capi.lib()
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    assert lib.pmoe_quantize_mx(x.data_ptr(), None, 4, x.data_ptr(), x.data_ptr(), 4, 48, None) == 1   # K % 32
    assert lib.pmoe_quantize_mx(None, None, 4, x.data_ptr(), x.data_ptr(), 4, 64, None) == 1
    lg = torch.zeros(4, 8, device=DEV)
    ids = torch.zeros(4, 9, dtype=torch.int32, device=DEV)
    assert lib.pmoe_route_topk(lg.data_ptr(), 0, 4, 8, 9, 1, ids.data_ptr(), ids.data_ptr(), None) == 2   # top_k > E
    assert lib.pmoe_route_topk(lg.data_ptr(), 7, 4, 8, 2, 1, ids.data_ptr(), ids.data_ptr(), None) == 1   # dtype code
    assert lib.pmoe_route_topk(lg.data_ptr(), 0, 4, 2000, 2, 1, ids.data_ptr(), ids.data_ptr(), None) == 2
