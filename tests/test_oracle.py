"""The CPU oracle against the golden vectors produced by the reference's own Python definitions
(tests/golden/make_golden.py), and the C restatement against the Python one. No GPU."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import build_ref, moe_oracle as O


@pytest.fixture(scope="module")
def clib():
    lib = C.CDLL(str(build_ref.build_c_oracle()))
    lib.oracle_moe_align.argtypes = [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p] * 3
    lib.oracle_pack_scales_blocked.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_int]
    lib.oracle_mx_quantize.argtypes = [C.c_void_p, C.c_long, C.c_int, C.c_void_p, C.c_void_p]
    return lib


def c_moe_align(clib, ids, E, block_m, bpc):
    ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    pad_to, max_padded, max_blocks = O.moe_align_sizes(ids.size, E, block_m, bpc)
    s = np.empty(max_padded, np.int32)
    e = np.empty(max_blocks, np.int32)
    n = np.empty(1, np.int32)
    rc = clib.oracle_moe_align(ids.ctypes.data, ids.size, E, block_m, pad_to, max_padded, max_blocks,
                               s.ctypes.data, e.ctypes.data, n.ctypes.data)
    assert rc == 0
    return s, e, n


def test_align_matches_reference_python(golden):
    """Exact-size tables of test/test.py:81-120: same counts, same blocks, same members per expert."""
    for case in golden["align"]:
        ids, E, bm = case["topk_ids"], case["num_experts"], case["block_m"]
        ref_s = case["sorted_token_ids"].numpy()
        ref_e = case["expert_ids"].numpy()
        ref_n = case["num_tokens_post_padded"].numpy()
        s, e, n = O.moe_align_spec(ids.numpy(), E, bm, 1)
        total = int(ref_n[0])
        assert int(n[0]) == total
        assert np.array_equal(e[: total // bm], ref_e)
        assert np.all(e[total // bm:] == E - 1)
        assert np.all(s[total:] == -1)
        canon_ref = O.canonical_alignment(ref_s, ref_e, ref_n, bm)
        assert np.array_equal(O.canonical_alignment(s[:total], e, n, bm), canon_ref)
        # the stable spec is already canonical
        assert np.array_equal(s[:total], canon_ref)
        s2, e2, n2 = O.moe_align_simple(ids, bm, E)
        assert np.array_equal(s2.numpy(), canon_ref) and np.array_equal(e2.numpy(), ref_e)


@pytest.mark.parametrize("T,E,k,bpc", [(1, 8, 2, 1), (300, 37, 9, 1), (1000, 128, 8, 2), (64, 1, 1, 1),
                                        (513, 1024, 4, 1), (0, 4, 2, 1)])
def test_align_c_equals_python(clib, T, E, k, bpc):
    g = torch.Generator().manual_seed(T + E)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).numpy()
    a = O.moe_align_spec(ids, E, 128, bpc)
    b = c_moe_align(clib, ids, E, 128, bpc)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_align_edge_cases(clib):
    # every pair on one expert; empty experts around it occupy no blocks
    ids = np.full((200, 2), 5, np.int32)
    s, e, n = O.moe_align_spec(ids, 8, 128, 1)
    assert int(n[0]) == 512 and list(e[:4]) == [5, 5, 5, 5] and np.all(e[4:] == 7)
    assert np.array_equal(s[:400], np.arange(400)) and np.all(s[400:] == -1)
    # ids outside [0, E) are ignored
    ids = np.array([[0, 9], [-1, 1]], np.int32)
    s, e, n = O.moe_align_spec(ids, 4, 128, 1)
    assert int(n[0]) == 256 and s[0] == 0 and s[128] == 3
    b = c_moe_align(clib, ids, 4, 128, 1)
    assert np.array_equal(b[0], s)
    # bpc = 2 pads to 256
    ids = np.zeros((3, 1), np.int32)
    s, e, n = O.moe_align_spec(ids, 2, 128, 2)
    assert int(n[0]) == 256 and list(e[:2]) == [0, 0]


def test_quantize_mx_golden(golden, clib):
    for case in golden["quant"]:
        t = case["input"]
        q, s = O.quantize_mx(t)
        assert torch.equal(q.view(torch.uint8), case["q"]), case["name"]
        assert torch.equal(s.view(torch.uint8), case["scales"]), case["name"]
        assert torch.equal(O.dequantize_mx(q, s), case["dequant"]), case["name"]
        # C restatement, bit for bit
        tf = t.float().contiguous().numpy()
        rows, k = tf.reshape(-1, tf.shape[-1]).shape
        cq = np.empty((rows, k), np.uint8)
        cs = np.empty((rows, k // 32), np.uint8)
        clib.oracle_mx_quantize(tf.ctypes.data, rows, k, cq.ctypes.data, cs.ctypes.data)
        assert np.array_equal(cs, case["scales"].numpy().reshape(rows, -1)), case["name"]
        assert np.array_equal(cq, case["q"].numpy().reshape(rows, -1)), case["name"]


def test_pack_scales_blocked_golden(golden, clib):
    for case in golden["pack"]:
        u = case["scales"]
        got = O.pack_scales_blocked(u.view(torch.float8_e8m0fnu)).view(torch.uint8)
        assert torch.equal(got, case["packed"])
        mn, kb = u.shape[-2:]
        lead = u.numel() // (mn * kb)
        out = np.empty(u.numel(), np.uint8)
        src = u.contiguous().numpy()
        clib.oracle_pack_scales_blocked(src.ctypes.data, out.ctypes.data, lead, mn, kb)
        assert np.array_equal(out, case["packed"].numpy().reshape(-1))


def test_pack_scales_is_a_permutation():
    idx = O.pack_scales_blocked_index(256, 8).reshape(-1)
    assert np.array_equal(np.sort(idx), np.arange(256 * 8))


def test_moe_reference_bf16_golden(golden):
    """moe_naive_from_topk of test/test.py:13-48, run by the generator on the same inputs."""
    for case in golden["moe_bf16"]:
        args = (case["x"], case["w1"], case["w2"], case["topk_ids"], case["topk_weights"])
        ref = case["out"].float()
        scale = ref.abs().max()
        a = O.moe_ref_grouped_mm(*args).float()
        b = O.moe_ref_bf16(*args).float()
        c = O.moe_ref_fp32(*args)
        # same op sequence: equal up to bf16 rounding of differently ordered fp32 sums
        assert (a - ref).abs().max() <= 2 ** -7 * scale
        assert (b - ref).abs().max() <= 2 ** -7 * scale
        # all-fp32 evaluation sits within the documented noise floor of the bf16 oracle
        assert O.max_rel_to_peak(c, ref) < 2e-2


def test_moe_reference_mxfp8_golden(golden):
    """moe_naive_from_topk of test/test_mxfp8.py:50-77 (activation requantised) on dequantised inputs."""
    for case in golden["moe_mxfp8"]:
        f8, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
        x = O.dequantize_mx(case["x_q"].view(f8), case["x_scales"].view(e8)).to(torch.bfloat16)
        w1 = O.dequantize_mx(case["w1_q"].view(f8), case["w1_scales"].view(e8)).to(torch.bfloat16)
        w2 = O.dequantize_mx(case["w2_q"].view(f8), case["w2_scales"].view(e8)).to(torch.bfloat16)
        ref = case["out"].float()
        scale = ref.abs().max()
        got = O.moe_ref_grouped_mm(x, w1, w2, case["topk_ids"], case["topk_weights"], requant_act=True).float()
        assert (got - ref).abs().max() <= 2 ** -6 * scale
        # quantising the fp32 activation (what the kernels do) instead of the bf16-rounded one (what the
        # reference's test oracle does) flips some e4m3 roundings: a few percent of the peak at most
        got32 = O.moe_ref_fp32(x, w1, w2, case["topk_ids"], case["topk_weights"], requant_act=True)
        assert O.max_rel_to_peak(got32, ref) < 5e-2


def test_routing_generators():
    ids, w = O.make_routing(64, 16, 4, 3, "uniform")
    assert ids.shape == (64, 4) and ids.dtype == torch.int32
    assert all(len(set(r.tolist())) == 4 for r in ids)
    assert torch.allclose(w.sum(-1), torch.ones(64))
    ids2, _ = O.make_routing(64, 16, 4, 3, "uniform")
    assert torch.equal(ids, ids2)
    z, _ = O.make_routing(2000, 128, 8, 3, "zipf")
    counts = torch.bincount(z.flatten().long(), minlength=128)
    assert all(len(set(r.tolist())) == 8 for r in z[:50])
    assert counts.max() > 8 * counts.float().median()   # heavy head


def test_backward_expert_slice_matches_autograd_oracle():
    """The slice-wise weight-gradient restatement equals autograd through the fp32 oracle."""
    T, K, E, N, k = 40, 64, 3, 128, 2
    H = N // 2
    x, w1, w2, ids, wts = O.make_case(T, K, E, N, k, seed=9)
    d_out = torch.randn(T, K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    _, d_w1, d_w2, _ = O.moe_backward_ref_fp32(x, w1, w2, ids, wts, d_out)
    for e in range(E):
        tok, route = torch.nonzero(ids == e, as_tuple=True)
        hs = slice(16, 48)
        got = O.moe_backward_expert_slice_ref(x[tok], d_out[tok], wts[tok, route], w1[e, hs], w1[e, H + 16:H + 48],
                                              w2[e][:, hs])
        for g, want in zip(got, (d_w1[e, hs], d_w1[e, H + 16:H + 48], d_w2[e][:, hs])):
            assert torch.allclose(g, want, rtol=1e-4, atol=1e-4)
