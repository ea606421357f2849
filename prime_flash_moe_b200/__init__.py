"""B200-native fused MoE FFN behind the ``prime_moe`` torch-library API.

Python surface of the reference package (prime_moe/__init__.py:27-49 ``fused_moe_bf16``, :75-100
``fused_moe_mxfp8``, :103 ``BLOCK``, :106-115 ``pack_scales_blocked``) plus ``moe_align`` (the
reference exposes it only as ``torch.ops.prime_moe.moe_align``). The operators are registered by
``_C.so`` (TORCH_LIBRARY fragment ``prime_moe``) which forwards to the C ABI of
``_lib/libpmoe_b200.so``. There is no CPU or eager fallback: importing this package without the
built libraries raises.
"""
from __future__ import annotations

from pathlib import Path

import torch

from . import _build

_PKG = Path(__file__).resolve().parent


def _load() -> None:
    missing = [p for p in (_build.NATIVE_LIB, _build.TORCH_EXT) if not p.exists()]
    if missing:
        raise ImportError(
            "prime_flash_moe_b200: native libraries not built ("
            + ", ".join(str(m.relative_to(_PKG.parent)) for m in missing)
            + "); run `python prime_flash_moe_b200/_build.py` (needs nvcc and g++)"
        )
    torch.ops.load_library(str(_build.TORCH_EXT))


_load()

BLOCK = 32  # MX scale block size (prime_moe/__init__.py:103)


@torch.library.register_fake("prime_moe::fused_moe_bf16")
def _fused_moe_bf16_fake(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, out,
                         top_k, block_m, block_n, warp_n, stages, bpc, cpc, split):
    return None


@torch.library.register_fake("prime_moe::fused_moe_mxfp8")
def _fused_moe_mxfp8_fake(x, x_scales, w, w_scales, w2, w2_scales, sorted_token_ids, expert_ids,
                          num_tokens_post_padded, topk_weights, out, top_k, block_m, block_n, warp_n, stages,
                          bpc, split):
    return None


@torch.library.register_fake("prime_moe::moe_align")
def _moe_align_fake(topk_ids, num_experts, block_m, bpc):
    n = topk_ids.numel()
    pad_to = block_m * bpc
    max_padded = (n + num_experts * (pad_to - 1) + pad_to - 1) // pad_to * pad_to
    mk = lambda k: topk_ids.new_empty((k,), dtype=torch.int32)
    return mk(max_padded), mk(max_padded // block_m), mk(1)


def fused_moe_bf16(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, out, top_k,
                   block_m, block_n, warp_n, stages, bpc=1, cpc=1, split=True):
    """In-place fused MoE FFN on bf16 operands; returns ``out`` (prime_moe/__init__.py:27-49).

    ``split=False`` accumulates into ``out`` (zero it first); ``split=True`` zeroes ``out`` itself.
    """
    torch.ops.prime_moe.fused_moe_bf16(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                       topk_weights, out, top_k, block_m, block_n, warp_n, stages, bpc, cpc,
                                       split)
    return out


def fused_moe_mxfp8(x, x_scales, w, w_scales, w2, w2_scales, sorted_token_ids, expert_ids,
                    num_tokens_post_padded, topk_weights, out, top_k, block_m, block_n, warp_n, stages, bpc=1,
                    split=True):
    """In-place fused MoE FFN on OCP-MX (e4m3 + e8m0/32) operands; returns ``out``
    (prime_moe/__init__.py:75-100). Weight scales must be in the ``pack_scales_blocked`` layout."""
    torch.ops.prime_moe.fused_moe_mxfp8(x, x_scales, w, w_scales, w2, w2_scales, sorted_token_ids, expert_ids,
                                        num_tokens_post_padded, topk_weights, out, top_k, block_m, block_n,
                                        warp_n, stages, bpc, split)
    return out


def moe_align(topk_ids, num_experts, block_m=128, bpc=1):
    """``(sorted_token_ids, expert_ids, num_tokens_post_padded)`` for ``topk_ids`` int32 ``(T, top_k)``
    (op schema prime_moe/csrc/torch_interface.cpp:316-322)."""
    return torch.ops.prime_moe.moe_align(topk_ids, num_experts, block_m, bpc)


def route_topk(logits, top_k, renormalize=True):
    """Router: logits ``[T, E]`` (fp32 or bf16) -> ``(topk_ids int32 [T, top_k], topk_weights fp32 [T, top_k])`` in
    one pass, experts by descending logit (ties to the lower index); ``renormalize`` = softmax over the selected
    logits, else the selected entries of the softmax over all experts. Not in the reference, which takes both
    tensors from the caller's gate (README.md:147)."""
    return torch.ops.prime_moe.route_topk(logits, top_k, renormalize)


def route_topk_align(logits, top_k, renormalize=True, block_m=128, bpc=1):
    """``route_topk`` and ``moe_align`` in one call: ``(topk_ids, topk_weights, sorted_token_ids, expert_ids,
    num_tokens_post_padded)``. Above the single-CTA sizes one kernel routes the tokens and counts its own ids per
    expert, so the histogram pass of ``moe_align`` and one launch disappear."""
    return torch.ops.prime_moe.route_topk_align(logits, top_k, renormalize, block_m, bpc)


def quantize_mx(x, row_index=None):
    """bf16 ``[T, K]`` -> OCP-MX ``(e4m3 [R, K], e8m0 [R, K/32])`` as ``fused_moe_mxfp8`` takes ``x`` / ``x_scales``;
    with ``row_index`` int32 ``[R]`` output row r is ``x[row_index[r]]``. Bit-identical to the reference's test
    quantiser (test/test_mxfp8.py:21-38), which the reference leaves to the caller (README.md:110-113)."""
    return torch.ops.prime_moe.quantize_mx(x, row_index)


def pack_scales_blocked(scales: torch.Tensor) -> torch.Tensor:
    """Row-major e8m0 scales ``(..., MN, K/32)`` -> the blocked layout the kernels read
    (prime_moe/__init__.py:106-115): 512-byte tiles covering 128 rows x 4 scale columns, tile index
    ``mn_tile * (K/128) + k_tile``, byte ``(r % 32) * 16 + (r // 32) * 4 + (kb % 4)`` inside a tile."""
    u = scales.view(torch.uint8)
    lead = u.shape[:-2]
    mn, kb = u.shape[-2:]
    assert mn % 128 == 0, f"MN ({mn}) must be a multiple of 128"
    assert kb % 4 == 0, f"K ({kb * 32}) must be a multiple of 128"
    tiles = u.reshape(-1, mn // 128, 4, 32, kb // 4, 4)     # (lead, mn_tile, r/32, r%32, k_tile, kb%4)
    tiles = tiles.permute(0, 1, 4, 3, 2, 5).contiguous()    # (lead, mn_tile, k_tile, r%32, r/32, kb%4)
    return tiles.reshape(*lead, -1).view(torch.float8_e8m0fnu)


def fused_moe_bf16_backward(x, w, w2, d_out, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, top_k,
                            gate_up=None):
    """Gradients of ``fused_moe_bf16`` (bpc = 1 routing tensors): ``(d_x, d_w, d_w2, d_topk_weights)``. ``gate_up`` is
    the tensor ``fused_moe_bf16_keep`` returned for the same inputs; without it the pre-activations are recomputed.
    The reference is forward-only (README.md:17); the checker is autograd through the fp32 test oracle
    (test/test.py:13-48)."""
    return torch.ops.prime_moe.fused_moe_bf16_backward(x, w, w2, d_out.contiguous(), sorted_token_ids, expert_ids,
                                                       num_tokens_post_padded, topk_weights, top_k, gate_up)


def fused_moe_bf16_keep(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, out, top_k,
                        bpc=1):
    """``fused_moe_bf16`` (split pipeline; ``bpc`` as ``moe_align`` was run) writing ``out`` and returning the gate/up
    pre-activations ``[sorted_num, N]`` its gate/up kernel saw, for ``fused_moe_bf16_backward(..., gate_up=...)``."""
    return torch.ops.prime_moe.fused_moe_bf16_keep(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                                   topk_weights, out, top_k, bpc)


class _MoEFFN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, w2, topk_ids, topk_weights, recompute):
        num_experts, top_k = w.shape[0], topk_ids.shape[1]
        bpc = 2 if w.shape[1] >= 8192 else 1        # CTA pairs pay off on wide layers (as in bench.py)
        sorted_ids, expert_ids, npp = torch.ops.prime_moe.moe_align(topk_ids, num_experts, 128, bpc)
        wts = topk_weights.detach().float().contiguous()
        out = torch.empty_like(x)
        gate_up = None
        if recompute:
            torch.ops.prime_moe.fused_moe_bf16(x, w, w2, sorted_ids, expert_ids, npp, wts, out, top_k, 128, 64, 4, 4, bpc,
                                               1, True)
        else:
            gate_up = fused_moe_bf16_keep(x, w, w2, sorted_ids, expert_ids, npp, wts, out, top_k, bpc)
        ctx.save_for_backward(x, w, w2, sorted_ids, expert_ids, npp, wts, gate_up)
        ctx.top_k = top_k
        ctx.weights_dtype = topk_weights.dtype
        return out

    @staticmethod
    def backward(ctx, d_out):
        x, w, w2, sorted_ids, expert_ids, npp, wts, gate_up = ctx.saved_tensors
        d_x, d_w, d_w2, d_wt = fused_moe_bf16_backward(x, w, w2, d_out, sorted_ids, expert_ids, npp, wts, ctx.top_k, gate_up)
        return d_x, d_w, d_w2, None, d_wt.to(ctx.weights_dtype), None


def moe_ffn(x, w, w2, topk_ids, topk_weights, recompute=False):
    """Differentiable bf16 MoE FFN layer: ``moe_align`` + ``fused_moe_bf16`` forward, ``fused_moe_bf16_backward`` for the
    gradients of ``x``, ``w``, ``w2`` and ``topk_weights``. The forward call keeps the gate/up pre-activations
    (``sorted_num * N`` bf16) for the backward pass; ``recompute=True`` keeps nothing and recomputes them there (one
    more GEMM of the gate/up size)."""
    return _MoEFFN.apply(x, w, w2, topk_ids, topk_weights, recompute)


__all__ = ["fused_moe_bf16", "fused_moe_mxfp8", "moe_align", "pack_scales_blocked", "route_topk", "route_topk_align", "quantize_mx",
           "fused_moe_bf16_backward", "fused_moe_bf16_keep", "moe_ffn", "BLOCK"]
