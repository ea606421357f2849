"""Backward pass of fused_moe_bf16 on the GPU against autograd through the all-fp32 CPU oracle.

Tolerance: max|grad - ref| <= 2e-2 * max|ref| per gradient tensor (the forward's tolerance; every intermediate of
the backward pass - gate/up pre-activations, activation, d_gate/d_up, d_xs - is rounded to bf16 once)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


def run_backward(x, w1, w2, ids, wts, d_out, need_weight_grad=True):
    from prime_flash_moe_b200 import capi
    E = w1.shape[0]
    k = ids.shape[1]
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, 1)
    grads = capi.fused_moe_bf16_backward(x.to(DEV), w1.to(DEV), w2.to(DEV), d_out.to(DEV), s, e, n, wts.to(DEV), k,
                                         need_weight_grad=need_weight_grad)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    return tuple(None if g is None else g.cpu() for g in grads)


def check(grads, refs):
    for name, g, r in zip(("d_x", "d_w1", "d_w2", "d_topk_weights"), grads, refs):
        if g is None:
            continue
        assert torch.isfinite(g.float()).all(), name
        err = O.max_rel_to_peak(g, r)
        assert err <= TOL, f"{name}: {err}"


@pytest.mark.parametrize("T,K,E,N,k", [
    (1, 128, 2, 256, 1), (8, 128, 1, 256, 1), (64, 512, 4, 512, 2),
    (130, 320, 5, 768, 3),       # K neither a multiple of 128 nor of 256: ragged row and column tiles
    (100, 256, 4, 384, 2),       # H = 192: ragged column tile of the SwiGLU step
    (256, 4096, 8, 512, 4),      # benchmark configuration 0
    (300, 1024, 8, 1024, 4), (1000, 384, 16, 256, 8),
])
def test_vs_autograd_of_fp32_oracle(T, K, E, N, k):
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=T + K)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    refs = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    check(run_backward(x, w1, w2, ids, wts, d_out), refs)


@pytest.mark.parametrize("pairs", ["0", "1", "2"])
def test_cta_pair_settings_agree_with_the_oracle(pairs, monkeypatch):
    # PMOE_BWD_PAIRS: 0 one-CTA kernel everywhere, 1 weight gradients on CTA pairs, 2 row-space GEMMs as well
    # (pairs of row blocks of one expert + the odd last blocks on the one-CTA kernel)
    monkeypatch.setenv("PMOE_BWD_PAIRS", pairs)
    T, K, E, N, k = 700, 384, 5, 768, 3       # 420 rows per expert: 3-4 row blocks each, odd and even counts
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=21)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    refs = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    check(run_backward(x, w1, w2, ids, wts, d_out), refs)


@pytest.mark.parametrize("pairs", ["0", "1"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_weight_gradients_in_fp32_and_accumulated(dtype, pairs, monkeypatch):
    """pmoe_fused_moe_bf16_backward_ex: fp32 weight gradients (tighter against the oracle than bf16 ones), and
    accumulation into what the tensors hold - two calls on a preset tensor give preset + 2 x gradient; experts
    without rows keep the preset."""
    from prime_flash_moe_b200 import capi
    monkeypatch.setenv("PMOE_BWD_PAIRS", pairs)
    T, K, E, N, k = 600, 384, 6, 512, 2
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=31)
    ids = (ids % 5).to(torch.int32)                       # expert 5 gets no rows
    ids[:, 1] = (ids[:, 0] + 1) % 5
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    refs = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, 1)
    args = (x.to(DEV), w1.to(DEV), w2.to(DEV), d_out.to(DEV), s, e, n, wts.to(DEV), k)
    plain = (torch.empty(E, N, K, dtype=dtype, device=DEV), torch.empty(E, K, N // 2, dtype=dtype, device=DEV))
    capi.fused_moe_bf16_backward(*args, d_w=plain)
    torch.cuda.synchronize()
    tol = 6e-3 if dtype == torch.float32 else TOL         # what is left is the bf16 rounding of d_gu / act
    assert O.max_rel_to_peak(plain[0].cpu(), refs[1]) <= tol and O.max_rel_to_peak(plain[1].cpu(), refs[2]) <= tol
    assert float(plain[0][5].float().abs().max()) == 0.0 and float(plain[1][5].float().abs().max()) == 0.0
    acc = (torch.full((E, N, K), 0.5, dtype=dtype, device=DEV), torch.full((E, K, N // 2), -0.25, dtype=dtype, device=DEV))
    for _ in range(2):
        capi.fused_moe_bf16_backward(*args, d_w=acc, accumulate=True)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for got, base, ref, preset in ((acc[0], plain[0], refs[1], 0.5), (acc[1], plain[1], refs[2], -0.25)):
        want = preset + 2 * base.float()
        scale = float(ref.abs().max())
        assert float((got.float() - want).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2) * max(scale, 1.0)
        assert float((got[5].float() - preset).abs().max()) == 0.0


def test_experts_without_rows_get_zero_weight_gradients():
    T, K, E, N, k = 8, 256, 16, 256, 2
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=3)
    ids = (ids % 3).to(torch.int32)           # only experts 0..2 are routed to
    ids[:, 1] = (ids[:, 0] + 1) % 3
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    refs = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    grads = run_backward(x, w1, w2, ids, wts, d_out)
    check(grads, refs)
    assert float(grads[1][3:].float().abs().max()) == 0.0
    assert float(grads[2][3:].float().abs().max()) == 0.0


def test_ids_out_of_range_are_ignored_and_weight_gradient_is_optional():
    T, K, E, N, k = 50, 256, 4, 256, 2
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=5)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    bad = ids.clone()
    bad[::7, 1] = E + 3                       # these routes are dropped by moe_align
    keep = bad < E
    refs = O.moe_backward_ref_fp32(x, w1, w2, torch.where(keep, bad, torch.zeros_like(bad)),
                                   torch.where(keep, wts, torch.zeros_like(wts)), d_out)
    grads = run_backward(x, w1, w2, bad, wts, d_out)
    check(grads[:3], refs[:3])
    assert float(grads[3][~keep].abs().max()) == 0.0
    assert O.max_rel_to_peak(grads[3][keep], refs[3][keep]) <= TOL
    assert run_backward(x, w1, w2, bad, wts, d_out, need_weight_grad=False)[3] is None


def test_argument_checks():
    from prime_flash_moe_b200 import capi
    x, w1, w2, ids, wts = O.make_case(16, 96, 2, 256, 1, seed=1)     # K = 96 is not a multiple of 64
    s, e, n = capi.moe_align(ids.to(DEV), 2, 128, 1)
    with pytest.raises(RuntimeError, match="multiple of 64"):
        capi.fused_moe_bf16_backward(x.to(DEV), w1.to(DEV), w2.to(DEV), x.to(DEV), s, e, n, wts.to(DEV), 1)
    x, w1, w2, ids, wts = O.make_case(16, 128, 2, 256, 1, seed=1)
    s, e, n = capi.moe_align(ids.to(DEV), 2, 128, 1)
    small = torch.empty(2048, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="workspace"):
        capi.fused_moe_bf16_backward(x.to(DEV), w1.to(DEV), w2.to(DEV), x.to(DEV), s, e, n, wts.to(DEV), 1,
                                     workspace=small[(-small.data_ptr()) % 1024:][:1024])


@pytest.mark.parametrize("bpc", [1, 2])
@pytest.mark.parametrize("T,K,E,N,k", [(64, 512, 4, 512, 2), (256, 4096, 8, 512, 4), (2100, 256, 2, 768, 1)])
def test_kept_pre_activations(T, K, E, N, k, bpc):
    """The forward call that keeps gate | up: same `out` as the plain call, the kept rows equal xs @ W1[e]^T, and the
    backward pass fed with them matches the oracle (the last shape has > 1024 rows per expert: the two-block
    gate/up kernel). bpc = 2: routing tables padded to 256 rows, CTA-pair gate/up kernel + single-block tails, and
    a backward pass that skips the blocks without routed rows."""
    from prime_flash_moe_b200 import capi
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=T + 3)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    s, e, n = capi.moe_align(ids.to(DEV), E, 128, bpc)
    dx, dw1, dw2, dwts = x.to(DEV), w1.to(DEV), w2.to(DEV), wts.to(DEV)
    plain = torch.empty(T, K, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_bf16(dx, dw1, dw2, s, e, n, dwts, plain, k, bpc=bpc)
    out, gate_up = capi.fused_moe_bf16_keep(dx, dw1, dw2, s, e, n, dwts, torch.empty_like(plain), k, bpc=bpc)
    torch.cuda.synchronize()
    assert O.max_rel_to_peak(out.cpu(), plain.cpu()) <= 1e-2     # bf16 reductions into `out` come in any order
    rows = s.cpu().long()
    live = torch.nonzero(rows >= 0).flatten()[:: max(1, T * k // 257)]          # a sample of the routed rows
    expert = e.cpu().long()[live // 128]
    want = torch.einsum("rk,rnk->rn", x.float()[rows[live] // k], w1.float()[expert])
    assert O.max_rel_to_peak(gate_up.cpu()[live], want) <= 1e-2
    assert torch.isfinite(gate_up[torch.nonzero(s >= 0).flatten()].float()).all()
    grads = capi.fused_moe_bf16_backward(dx, dw1, dw2, d_out.to(DEV), s, e, n, dwts, k, gate_up=gate_up)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    check(tuple(g.cpu() for g in grads), O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out))


@pytest.mark.parametrize("recompute", [False, True])
def test_autograd_layer_matches_oracle_gradients(recompute):
    import prime_flash_moe_b200 as P
    T, K, E, N, k = 200, 512, 6, 512, 3
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=11)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    refs = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    leaves = [t.to(DEV).requires_grad_(True) for t in (x, w1, w2, wts)]
    out = P.moe_ffn(leaves[0], leaves[1], leaves[2], ids.to(DEV), leaves[3], recompute=recompute)
    assert O.max_rel_to_peak(out.detach().cpu(), O.moe_ref_fp32(x, w1, w2, ids, wts)) <= TOL
    out.backward(d_out.to(DEV))
    torch.cuda.synchronize()
    check(tuple(t.grad.cpu() for t in leaves), refs)
