"""CPU oracle for the fused MoE FFN hot path. TEST INFRASTRUCTURE ONLY.

Nothing in the product (``prime_flash_moe_b200``) imports this module; only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg may. It restates, on the host and in
plain torch/numpy, what the reference computes on the path

    moe_align -> gate/up GEMM -> SwiGLU (-> mxfp8 requant) -> down GEMM -> top-k weighted reduce

Pinning: the functions below are checked in ``tests/test_oracle.py`` against fixtures under
``tests/golden/`` that were produced by executing the reference's own Python definitions
(``test/test.py``, ``test/test_mxfp8.py``, ``prime_moe/__init__.py``) on the CPU; the script that made
them is ``tests/golden/make_golden.py``. On a GPU the CUDA kernels are additionally compared with the
reference's own sm_100a kernels compiled into ``oracle/_ref`` when that build is present.

Each function cites the reference lines it follows (paths inside PrimeIntellect-ai/prime-flash-moe).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

BLOCK = 32          # MX scale block (prime_moe/__init__.py:103)
E4M3_MAX = 448.0    # test/test_mxfp8.py:17
E4M3_EMAX = 8       # test/test_mxfp8.py:18  (448 = 1.75 * 2**8)


# ---------------------------------------------------------------------------------------------
# moe_align
# ---------------------------------------------------------------------------------------------
def moe_align_sizes(n: int, num_experts: int, block_m: int, bpc: int):
    """Upper-bound output sizes (prime_moe/csrc/torch_interface.cpp:88-91)."""
    pad_to = block_m * bpc
    max_padded = (n + num_experts * (pad_to - 1) + pad_to - 1) // pad_to * pad_to
    return pad_to, max_padded, max_padded // block_m


def moe_align_spec(topk_ids, num_experts: int, block_m: int = 128, bpc: int = 1):
    """The three outputs of ``moe_align`` at their full allocated sizes, with the order inside an
    expert fixed to ascending pair id.

    Follows the kernel prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu:853-907: histogram (:873-874),
    padded exclusive scan (:876-882), -1 fill (:885-886), ``expert_ids`` by "largest e with
    offs[e] <= row", ``E-1`` past the end (:887-900), scatter (:902-906; the reference's order inside
    an expert is whatever its atomics produce, this spec picks the stable one).
    Returns int32 numpy arrays ``(sorted_token_ids, expert_ids, num_tokens_post_padded)``.
    """
    ids = np.asarray(topk_ids, dtype=np.int64).reshape(-1)
    n = ids.size
    pad_to, max_padded, max_blocks = moe_align_sizes(n, num_experts, block_m, bpc)
    valid = (ids >= 0) & (ids < num_experts)
    counts = np.bincount(ids[valid], minlength=num_experts)
    padded = (counts + pad_to - 1) // pad_to * pad_to
    offs = np.zeros(num_experts + 1, dtype=np.int64)
    np.cumsum(padded, out=offs[1:])
    total = int(offs[-1])
    sorted_ids = np.full(max_padded, -1, dtype=np.int32)
    order = np.argsort(ids[valid], kind="stable")
    pair = np.nonzero(valid)[0][order]
    exp_sorted = ids[valid][order]
    starts = np.zeros(num_experts + 1, dtype=np.int64)
    np.cumsum(counts, out=starts[1:])
    rank = np.arange(pair.size) - starts[exp_sorted]
    sorted_ids[offs[exp_sorted] + rank] = pair.astype(np.int32)
    rows = np.arange(max_blocks, dtype=np.int64) * block_m
    # largest e in [0, E-1] with offs[e] <= row
    e = np.searchsorted(offs[:num_experts], rows, side="right") - 1
    expert_ids = np.where(rows >= total, num_experts - 1, np.clip(e, 0, num_experts - 1)).astype(np.int32)
    return sorted_ids, expert_ids, np.array([total], dtype=np.int32)


def moe_align_simple(topk_ids: torch.Tensor, block_m: int, num_experts: int):
    """Exact-size routing tables as the reference's tests build them (test/test.py:81-120,
    test/test_mxfp8.py:80-109): no tail padding, one run of ``ceil(count/block_m)*block_m`` rows per
    expert. Order inside an expert: ascending pair id (the tests use an unstable argsort)."""
    ids = topk_ids.reshape(-1).to(torch.int64).cpu().numpy()
    counts = np.bincount(ids, minlength=num_experts)
    padded = (counts + block_m - 1) // block_m * block_m
    order = np.argsort(ids, kind="stable")
    out, experts = [], []
    pos = 0
    for e in range(num_experts):
        c, pc = int(counts[e]), int(padded[e])
        out.append(order[pos:pos + c].astype(np.int32))
        out.append(np.full(pc - c, -1, dtype=np.int32))
        experts.extend([e] * (pc // block_m))
        pos += c
    sorted_ids = np.concatenate(out) if out else np.zeros(0, np.int32)
    dev = topk_ids.device
    return (torch.from_numpy(sorted_ids).to(dev), torch.tensor(experts, dtype=torch.int32, device=dev),
            torch.tensor([int(padded.sum())], dtype=torch.int32, device=dev))


def canonical_alignment(sorted_ids, expert_ids, npp, block_m: int):
    """Order-insensitive canonical form used to compare two ``moe_align`` results bit for bit: inside
    each run of blocks owned by one expert the valid ids are sorted ascending and the -1 padding is
    moved behind them; everything else is left untouched."""
    s = np.array(sorted_ids, dtype=np.int64).copy()
    e = np.asarray(expert_ids)
    total = int(np.asarray(npp).reshape(-1)[0])
    nb = total // block_m
    start = 0
    while start < nb:
        stop = start
        while stop < nb and e[stop] == e[start]:
            stop += 1
        seg = s[start * block_m:stop * block_m]
        key = np.where(seg < 0, np.iinfo(np.int64).max, seg)
        s[start * block_m:stop * block_m] = seg[np.argsort(key, kind="stable")]
        start = stop
    return s.astype(np.int32)


# ---------------------------------------------------------------------------------------------
# pack_scales_blocked
# ---------------------------------------------------------------------------------------------
def pack_scales_blocked_index(mn: int, kb: int) -> np.ndarray:
    """Destination byte offset of scale (r, k) of one ``(mn, kb)`` matrix in the blocked layout
    (prime_moe/__init__.py:106-115): tile ``(r//128)*(kb//4) + k//4``, byte
    ``(r%32)*16 + ((r%128)//32)*4 + k%4`` inside the 512-byte tile."""
    r = np.arange(mn)[:, None]
    k = np.arange(kb)[None, :]
    tile = (r // 128) * (kb // 4) + k // 4
    return tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + k % 4


def pack_scales_blocked(scales: torch.Tensor) -> torch.Tensor:
    u = scales.view(torch.uint8)
    *lead, mn, kb = u.shape
    assert mn % 128 == 0 and kb % 4 == 0
    idx = torch.from_numpy(pack_scales_blocked_index(mn, kb).reshape(-1))
    flat = u.reshape(-1, mn * kb)
    out = torch.empty_like(flat)
    out[:, idx] = flat
    return out.reshape(*lead, mn * kb).view(torch.float8_e8m0fnu)


# ---------------------------------------------------------------------------------------------
# OCP-MX quantiser
# ---------------------------------------------------------------------------------------------
def shared_exponent(amax: torch.Tensor) -> torch.Tensor:
    """Biased e8m0 exponent of a block with absolute maximum ``amax`` (test/test_mxfp8.py:21-24):
    the fp32 exponent field minus 8, clamped to [0, 254]."""
    bits = amax.float().contiguous().view(torch.int32)
    return (((bits >> 23) & 0xFF) - E4M3_EMAX).clamp(0, 254)


def quantize_mx(t: torch.Tensor, block: int = BLOCK):
    """``t`` -> (e4m3 values, e8m0 scales over the last dim) (test/test_mxfp8.py:27-38)."""
    k = t.shape[-1]
    assert k % block == 0
    g = t.float().reshape(*t.shape[:-1], k // block, block)
    e = shared_exponent(g.abs().amax(-1))
    inv = torch.exp2((127 - e).float())
    q = (g * inv.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(*t.shape[:-1], k).contiguous(), e.to(torch.uint8).view(torch.float8_e8m0fnu)


def dequantize_mx(q: torch.Tensor, scales: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    """fp32 values of an MX tensor (test/test_mxfp8.py:41-47)."""
    k = q.shape[-1]
    e = scales.view(torch.uint8).to(torch.int32)
    g = q.float().reshape(*q.shape[:-1], k // block, block) * torch.exp2((e - 127).float()).unsqueeze(-1)
    return g.reshape(*q.shape[:-1], k)


# ---------------------------------------------------------------------------------------------
# MoE references
# ---------------------------------------------------------------------------------------------
def _sorted_pairs(topk_ids: torch.Tensor, num_experts: int):
    flat = topk_ids.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, counts


def moe_ref_bf16(x, w1, w2, topk_ids, topk_weights, requant_act: bool = False):
    """The reference's own test oracle (test/test.py:13-48; with ``requant_act`` the mxfp8 variant
    test/test_mxfp8.py:50-77, whose only difference is the MX quantise->dequantise of the activation,
    :70-72): per-expert GEMMs with bf16 outputs, SwiGLU in fp32 rounded to bf16, routing weight
    applied in fp32, rounded to bf16, summed into a bf16 ``out`` in sorted-pair order."""
    T, K = x.shape
    E, N, _ = w1.shape
    top_k = topk_ids.shape[1]
    order, counts = _sorted_pairs(topk_ids, E)
    tok = order // top_k
    xs = x[tok]
    scale = topk_weights.reshape(-1)[order].float()
    y = torch.empty((order.numel(), K), dtype=torch.bfloat16)
    pos = 0
    for e in range(E):
        c = int(counts[e])
        if c == 0:
            continue
        h = (xs[pos:pos + c].float() @ w1[e].float().t()).to(torch.bfloat16)   # grouped_mm, bf16 out
        gate, up = h.chunk(2, dim=-1)
        act = (F.silu(gate.float()) * up.float()).to(torch.bfloat16)
        if requant_act:
            aq, asf = quantize_mx(act)
            act = dequantize_mx(aq, asf).to(torch.bfloat16)
        y[pos:pos + c] = (act.float() @ w2[e].float().t()).to(torch.bfloat16)
        pos += c
    y = (y.float() * scale[:, None]).to(torch.bfloat16)
    out = torch.zeros((T, K), dtype=torch.bfloat16)
    out.index_add_(0, tok, y)
    return out


def moe_ref_fp32(x, w1, w2, topk_ids, topk_weights, requant_act: bool = False):
    """All-fp32 evaluation of the same contraction (no intermediate bf16 rounding). With
    ``requant_act`` the fp32 SwiGLU output goes through the MX quantiser first, which is what the
    reference's fused mxfp8 kernel does on chip (prime_moe/csrc/kernels/fused_moe_mxfp8_kernel.cu
    :4-20, :375-403)."""
    T, K = x.shape
    E = w1.shape[0]
    top_k = topk_ids.shape[1]
    order, counts = _sorted_pairs(topk_ids, E)
    tok = order // top_k
    xs = x.float()[tok]
    scale = topk_weights.reshape(-1)[order].float()
    out = torch.zeros((T, K), dtype=torch.float32)
    pos = 0
    for e in range(E):
        c = int(counts[e])
        if c == 0:
            continue
        h = xs[pos:pos + c] @ w1[e].float().t()
        gate, up = h.chunk(2, dim=-1)
        act = F.silu(gate) * up
        if requant_act:
            aq, asf = quantize_mx(act)
            act = dequantize_mx(aq, asf)
        y = (act @ w2[e].float().t()) * scale[pos:pos + c, None]
        out.index_add_(0, tok[pos:pos + c], y)
        pos += c
    return out


def moe_ref_grouped_mm(x, w1, w2, topk_ids, topk_weights, requant_act: bool = False):
    """Line-by-line restatement of test/test.py:13-48 on ``torch._grouped_mm`` (CPU build of torch
    supports it); used to pin ``moe_ref_bf16`` and as the timed CPU baseline."""
    T, K = x.shape
    E, N, _ = w1.shape
    top_k = topk_ids.shape[1]
    flat = topk_ids.reshape(-1).to(torch.int32)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat[order], minlength=E).to(torch.int64)
    offs = torch.cumsum(counts, 0).to(torch.int32)
    tok = order // top_k
    scale = topk_weights.reshape(-1)[order].float()
    h = torch._grouped_mm(x[tok], w1.transpose(1, 2).contiguous(), offs, out_dtype=torch.bfloat16)
    gate, up = h.chunk(2, dim=-1)
    act = (F.silu(gate.float()) * up.float()).to(torch.bfloat16)
    if requant_act:
        aq, asf = quantize_mx(act)
        act = dequantize_mx(aq, asf).to(torch.bfloat16)
    y = torch._grouped_mm(act, w2.transpose(1, 2).contiguous(), offs, out_dtype=torch.bfloat16)
    y = (y.float() * scale[:, None]).to(torch.bfloat16)
    out = torch.zeros((T, K), dtype=torch.bfloat16)
    out.index_add_(0, tok.long(), y)
    return out


def rel_clamp(out: torch.Tensor, ref: torch.Tensor, floor: float) -> float:
    """The reference's accuracy metric ``max |d| / max(|ref|, floor)`` (test/test.py:172-176)."""
    d = (out.float() - ref.float()).abs()
    return float((d / ref.float().abs().clamp_min(floor)).max())


def max_rel_to_peak(out: torch.Tensor, ref: torch.Tensor) -> float:
    """``max|out - ref| / max|ref|`` - the gate used for parity with the fp32 oracle."""
    return float((out.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-30))


# ---------------------------------------------------------------------------------------------
# seeded synthetic inputs (the benchmark configurations)
# ---------------------------------------------------------------------------------------------
def make_routing(T: int, E: int, top_k: int, seed: int, dist: str = "uniform", zipf_s: float = 1.2):
    """``topk_ids`` int32 (T, top_k) with distinct experts per token and fp32 ``topk_weights`` =
    softmax of N(0,1) logits. ``dist='zipf'``: experts drawn without replacement with probability
    proportional to (rank+1)^-s over a seeded permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        ids = torch.rand(T, E, generator=g).argsort(-1)[:, :top_k]
    elif dist == "zipf":
        p = (torch.arange(E, dtype=torch.float64) + 1).pow(-zipf_s)
        perm = torch.randperm(E, generator=g)
        probs = torch.empty(E, dtype=torch.float64)
        probs[perm] = p / p.sum()
        ids = torch.multinomial(probs.expand(T, E), top_k, replacement=False, generator=g)
    else:
        raise ValueError(dist)
    weights = torch.softmax(torch.randn(T, top_k, generator=g), dim=-1)
    return ids.to(torch.int32).contiguous(), weights.float().contiguous()


def make_case(T, K, E, N, top_k, seed, dist="uniform", x_std=1.0, w_std=None):
    """Seeded bf16 problem: x ~ N(0, x_std^2), w1 ~ N(0, 1/K), w2 ~ N(0, 1/H) unless ``w_std``."""
    g = torch.Generator().manual_seed(seed)
    H = N // 2
    x = (torch.randn(T, K, generator=g) * x_std).to(torch.bfloat16)
    s1 = w_std if w_std is not None else K ** -0.5
    s2 = w_std if w_std is not None else H ** -0.5
    w1 = (torch.randn(E, N, K, generator=g) * s1).to(torch.bfloat16)
    w2 = (torch.randn(E, K, H, generator=g) * s2).to(torch.bfloat16)
    ids, wts = make_routing(T, E, top_k, seed + 1, dist)
    return x, w1, w2, ids, wts


def moe_backward_ref_fp32(x, w1, w2, topk_ids, topk_weights, d_out):
    """Gradients of the fp32 evaluation above (``moe_ref_fp32``, i.e. the contraction of the reference's test
    oracle test/test.py:13-48) with respect to ``x``, ``w1``, ``w2`` and ``topk_weights`` for an output gradient
    ``d_out``, by autograd. The reference has no backward pass (README.md:17); this is the checker of the
    library's own one. Returns fp32 ``(d_x, d_w1, d_w2, d_topk_weights)``."""
    leaves = [t.detach().float().clone().requires_grad_(True) for t in (x, w1, w2, topk_weights)]
    out = moe_ref_fp32(leaves[0], leaves[1], leaves[2], topk_ids, leaves[3])
    out.backward(d_out.float())
    return tuple(t.grad if t.grad is not None else torch.zeros_like(t) for t in leaves)


def moe_backward_expert_slice_ref(x_e, d_out_e, wt_e, w1_gate_rows, w1_up_rows, w2_cols):
    """Weight gradients of ONE expert restricted to a slice ``hs`` of its hidden columns, in fp32, from the rows routed
    to it: ``x_e`` [n, K], ``d_out_e`` [n, K] (gradient of the output rows of those tokens), ``wt_e`` [n] routing
    weights, ``w1_gate_rows`` = W1[e][hs], ``w1_up_rows`` = W1[e][H + hs] (both [h, K]), ``w2_cols`` = W2[e][:, hs]
    ([K, h]). Returns ``(d_W1[e][hs], d_W1[e][H + hs], d_W2[e][:, hs])``. Same contraction as
    ``moe_backward_ref_fp32`` (the test suite checks one against the other); exists so that full-size layers can be
    checked a slice at a time."""
    x_e, d_out_e, wt_e = x_e.float(), d_out_e.float(), wt_e.float()
    g = x_e @ w1_gate_rows.float().t()
    u = x_e @ w1_up_rows.float().t()
    s = torch.sigmoid(g)
    act = g * s * u
    c = d_out_e @ w2_cols.float()
    d_act = c * wt_e[:, None]
    d_gate = d_act * u * s * (1 + g * (1 - s))
    d_up = d_act * g * s
    return d_gate.t() @ x_e, d_up.t() @ x_e, d_out_e.t() @ (act * wt_e[:, None])
