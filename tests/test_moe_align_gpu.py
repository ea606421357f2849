"""moe_align on the GPU, through the C ABI and through the torch operator, bit-exact against the CPU
spec; and against the reference's own kernel (oracle/_ref) in canonical form when that build exists."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O, ref_kernels as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_capi(ids, E, block_m=128, bpc=1):
    from prime_flash_moe_b200 import capi
    s, e, n = capi.moe_align(ids.to(DEV), E, block_m, bpc)
    torch.cuda.synchronize()
    return s.cpu().numpy(), e.cpu().numpy(), n.cpu().numpy()


def _assert_exact(got, ids, E, block_m=128, bpc=1):
    ref = O.moe_align_spec(ids.numpy(), E, block_m, bpc)
    for name, a, b in zip(("sorted_token_ids", "expert_ids", "num_tokens_post_padded"), got, ref):
        assert a.shape == b.shape, name
        assert np.array_equal(a, b), f"{name} differs at {np.nonzero(a != b)[0][:8]}"


CASES = [
    # T, E, top_k, bpc, dist         (n = T*top_k; n <= 4096 takes the single-CTA path)
    (1, 8, 2, 1, "uniform"), (7, 4, 4, 1, "uniform"), (256, 8, 4, 1, "uniform"), (256, 8, 4, 2, "uniform"),
    (1, 128, 8, 1, "uniform"), (16, 128, 8, 1, "uniform"), (128, 128, 8, 1, "uniform"),
    (512, 128, 8, 1, "uniform"), (513, 128, 8, 1, "uniform"),
    (1024, 128, 8, 1, "uniform"), (8192, 128, 8, 1, "uniform"), (32768, 128, 8, 1, "uniform"),
    (4096, 8, 2, 1, "uniform"), (4096, 8, 2, 2, "uniform"),
    (16384, 256, 8, 1, "uniform"), (65536, 128, 8, 1, "zipf"), (65536, 128, 8, 2, "zipf"),
    (3000, 1024, 8, 1, "uniform"), (5000, 1, 1, 1, "uniform"), (777, 37, 9, 1, "zipf"),
    (40000, 1024, 8, 1, "uniform"), (20000, 300, 8, 1, "zipf"), (9000, 3, 2, 1, "uniform"),   # one CTA per SM; odd E
]


@pytest.mark.parametrize("T,E,k,bpc,dist", CASES)
def test_bit_exact_vs_spec(T, E, k, bpc, dist):
    ids, _ = O.make_routing(T, E, k, seed=T + E + k, dist=dist)
    _assert_exact(_run_capi(ids, E, 128, bpc), ids, E, 128, bpc)


def test_reference_sweep_routing_with_duplicates():
    """Routing of the reference's test sweeps (test/test.py:155-156): top_k-1 experts drawn WITH
    replacement from E-1 experts plus the last expert forced, so duplicates per token are legal."""
    g = torch.Generator().manual_seed(5)
    for T in (8, 32, 128, 256, 2000):
        for E in (257, 8, 37):
            ids = torch.randint(0, E - 1, (T, 9), generator=g, dtype=torch.int32)
            ids[:, -1] = E - 1
            _assert_exact(_run_capi(ids, E), ids, E)


def test_edge_cases():
    one = torch.full((1000, 4), 3, dtype=torch.int32)          # all pairs on one expert
    _assert_exact(_run_capi(one, 16), one, 16)
    big_one = torch.full((5000, 4), 0, dtype=torch.int32)       # same, multi-CTA path
    _assert_exact(_run_capi(big_one, 16), big_one, 16)
    bad = torch.tensor([[0, 99], [-5, 1], [2, 2]], dtype=torch.int32)   # out-of-range ids are ignored
    _assert_exact(_run_capi(bad, 4), bad, 4)
    g = torch.Generator().manual_seed(1)
    bad_big = torch.randint(-3, 20, (4000, 4), generator=g, dtype=torch.int32)
    _assert_exact(_run_capi(bad_big, 16), bad_big, 16)
    odd = torch.randint(0, 5, (100, 3), generator=g, dtype=torch.int32)  # block_m other than 128
    _assert_exact(_run_capi(odd, 5, 16, 3), odd, 5, 16, 3)


def test_deterministic_and_reentrant():
    ids, _ = O.make_routing(20000, 64, 8, seed=2, dist="zipf")
    a = _run_capi(ids, 64)
    for _ in range(3):
        b = _run_capi(ids, 64)
        assert all(np.array_equal(x, y) for x, y in zip(a, b))


def test_torch_operator_and_workspace_variant():
    import prime_flash_moe_b200 as P
    from prime_flash_moe_b200 import capi
    ids, _ = O.make_routing(9000, 128, 8, seed=3)
    s, e, n = P.moe_align(ids.to(DEV), 128, 128, 1)
    _assert_exact((s.cpu().numpy(), e.cpu().numpy(), n.cpu().numpy()), ids, 128)
    s, e, n = torch.ops.prime_moe.moe_align(ids.to(DEV), 128, 128, 2)
    _assert_exact((s.cpu().numpy(), e.cpu().numpy(), n.cpu().numpy()), ids, 128, 128, 2)
    with pytest.raises(RuntimeError):
        torch.ops.prime_moe.moe_align(ids.to(DEV), 2000, 128, 1)       # > 1024 experts
    with pytest.raises(RuntimeError):
        torch.ops.prime_moe.moe_align(ids.to(DEV).long(), 128, 128, 1)  # dtype check
    assert capi.device_status() == 0


@pytest.mark.skipif(not R.available(), reason="oracle/_ref (reference kernels) not built")
@pytest.mark.parametrize("T,E,k,bpc,dist", [(256, 8, 4, 1, "uniform"), (1, 128, 8, 1, "uniform"),
                                             (8192, 128, 8, 1, "uniform"), (65536, 128, 8, 1, "zipf"),
                                             (16384, 256, 8, 2, "uniform"), (300, 257, 9, 1, "uniform")])
def test_equals_reference_kernel(T, E, k, bpc, dist):
    """num_tokens_post_padded and expert_ids equal bit for bit over their full allocated length;
    sorted_token_ids equal after sorting inside each expert's padded segment (the reference's order
    there depends on its atomics)."""
    ids, _ = O.make_routing(T, E, k, seed=11 + T, dist=dist)
    mine = _run_capi(ids, E, 128, bpc)
    rs, re_, rn = R.moe_align(ids.to(DEV), E, 128, bpc)
    torch.cuda.synchronize()
    rs, re_, rn = rs.cpu().numpy(), re_.cpu().numpy(), rn.cpu().numpy()
    assert np.array_equal(mine[2], rn)
    assert np.array_equal(mine[1], re_)
    assert np.array_equal(O.canonical_alignment(mine[0], mine[1], mine[2], 128),
                          O.canonical_alignment(rs, re_, rn, 128))
