"""ctypes view of the C ABI (``include/pmoe_b200.h``) for callers that hold raw device pointers.

The functions here take torch tensors only to read ``data_ptr()`` and the current CUDA stream; they
call ``libpmoe_b200.so`` directly, bypassing the torch operator registration. A non-zero status is
raised as ``RuntimeError`` carrying ``pmoe_last_error()``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

from . import _build

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t

# name -> (restype, argtypes); mirrors include/pmoe_b200.h declaration by declaration
SIGNATURES = {
    "pmoe_last_error": (C.c_char_p, []),
    "pmoe_version": (_i, []),
    "pmoe_moe_align": (_i, [_vp] * 4 + [_i] * 6 + [_vp]),
    "pmoe_moe_align_workspace_bytes": (_sz, [_i, _i]),
    "pmoe_moe_align_ws": (_i, [_vp] * 4 + [_i] * 6 + [_vp, _sz, _vp]),
    "pmoe_moe_align_static": (_i, [_vp] * 4 + [_i] * 6 + [_vp]),
    "pmoe_moe_align_static_capacity_bytes": (_sz, []),
    "pmoe_fused_moe_bf16": (_i, [_vp] * 8 + [_i] * 13 + [_vp]),
    "pmoe_fused_moe_bf16_workspace_bytes": (_sz, [_i] * 5),
    "pmoe_fused_moe_bf16_ws": (_i, [_vp] * 8 + [_i] * 13 + [_vp, _sz, _vp]),
    "pmoe_fused_moe_bf16_ex": (_i, [_vp] * 8 + [_i] * 13 + [_vp, _sz, _vp, _vp, _vp]),
    "pmoe_fused_moe_mxfp8_ex": (_i, [_vp] * 11 + [_i] * 12 + [_vp, _sz, _vp, _vp]),
    "pmoe_ep_return_table": (_i, [_vp, _sz, _i, _i, _i, _i, _i, _vp, _vp]),
    "pmoe_fused_moe_mxfp8": (_i, [_vp] * 11 + [_i] * 12 + [_vp]),
    "pmoe_fused_moe_mxfp8_workspace_bytes": (_sz, [_i] * 5),
    "pmoe_fused_moe_mxfp8_ws": (_i, [_vp] * 11 + [_i] * 12 + [_vp, _sz, _vp]),
    "pmoe_ep_plan_workspace_bytes": (C.c_size_t, [_i, _i]),
    "pmoe_ep_plan": (_i, [_vp] * 2 + [_i] * 4 + [_vp] * 5 + [C.c_size_t, _vp]),
    "pmoe_ep_combine": (_i, [_vp] * 3 + [_i] * 3 + [_vp]),
    "pmoe_device_status": (_i, [C.POINTER(_i)]),
    "pmoe_reset_device_status": (_i, []),
    "pmoe_debug_set_phase_mask": (_i, [_i]),
    "pmoe_debug_set_l2_ahead": (_i, [_i]),
    "pmoe_ep_header_bytes": (_sz, []),
    "pmoe_ep_buffer_alloc": (_i, [_sz, C.POINTER(_vp), _vp]),
    "pmoe_ep_buffer_open": (_i, [_vp, C.POINTER(_vp)]),
    "pmoe_ep_buffer_close": (_i, [_vp]),
    "pmoe_ep_buffer_free": (_i, [_vp]),
    "pmoe_ep_publish_counts": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "pmoe_ep_push_rows": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _vp, _sz, _sz, _sz, _i, _i, _i, _i, _vp]),
    "pmoe_ep_recv_prepare": (_i, [_vp, _sz, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pmoe_ep_push_back": (_i, [_vp, _i, _vp, _sz, _i, _i, _i, _i, _i, _vp]),
    "pmoe_ep_combine_peer": (_i, [_vp, _sz, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pmoe_route_topk": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "pmoe_route_topk_align": (_i, [_vp, _i, _i, _i, _i, _i] + [_vp] * 5 + [_i] * 4 + [_vp, _sz, _vp]),
    "pmoe_quantize_mx": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _vp]),
    "pmoe_fused_moe_bf16_backward_workspace_bytes": (_sz, [_i] * 6),
    "pmoe_fused_moe_bf16_backward": (_i, [_vp] * 8 + [_i] * 6 + [_vp] * 6 + [_sz, _vp]),
    "pmoe_fused_moe_bf16_backward_ex": (_i, [_vp] * 8 + [_i] * 6 + [_vp] * 5 + [_i, _i, _vp, _sz, _vp]),
    "pmoe_fused_moe_bf16_keep_ws": (_i, [_vp] * 8 + [_i] * 7 + [_vp, _vp, _sz, _vp]),
    "pmoe_debug_set_backward_mask": (_i, [_i]),
    "pmoe_debug_set_wait_ns": (_i, [C.c_ulonglong]),
    "pmoe_debug_wait_probe": (_i, [_vp]),
    "pmoe_debug_bf16_workspace_extent": (_sz, [_i] * 8),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded shared library with argtypes/restypes set. Raises if it was not built."""
    global _lib
    if _lib is None:
        path = Path(_build.NATIVE_LIB)
        if not path.exists():
            raise ImportError(f"{path} not built; run `python prime_flash_moe_b200/_build.py`")
        handle = C.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if a declared symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(lib().pmoe_last_error().decode() or f"pmoe status {rc}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t) -> int:
    return 0 if t is None else t.data_ptr()


def moe_align(topk_ids: torch.Tensor, num_experts: int, block_m: int = 128, bpc: int = 1):
    assert topk_ids.is_cuda and topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
    n = topk_ids.numel()
    pad_to = block_m * bpc
    max_padded = (n + num_experts * (pad_to - 1) + pad_to - 1) // pad_to * pad_to
    max_blocks = max_padded // block_m
    mk = lambda k: torch.empty(k, dtype=torch.int32, device=topk_ids.device)
    sorted_ids, expert_ids, npp = mk(max_padded), mk(max_blocks), mk(1)
    with torch.cuda.device(topk_ids.device):
        _check(lib().pmoe_moe_align(_p(topk_ids), _p(sorted_ids), _p(expert_ids), _p(npp), n, num_experts,
                                    block_m, pad_to, max_padded, max_blocks, _stream()))
    return sorted_ids, expert_ids, npp


def _workspace(nbytes, device):
    ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
    off = (-ws.data_ptr()) % 1024
    return ws[off:off + nbytes]


def fused_moe_bf16(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, out, top_k,
                   block_m=128, block_n=64, warp_n=4, stages=4, bpc=1, cpc=1, split=True, workspace=None,
                   live_rows=None, out_rows=None):
    M, K = x.shape
    E, N, _ = w.shape
    with torch.cuda.device(x.device):
        common = (_p(x), _p(w), _p(w2), _p(out), _p(sorted_token_ids), _p(expert_ids), _p(num_tokens_post_padded),
                  _p(topk_weights), top_k, M, K, N, E, sorted_token_ids.numel(), block_m, block_n, warp_n, stages,
                  bpc, cpc, int(split))
        if live_rows is not None or out_rows is not None:
            if workspace is None:
                workspace = _workspace(lib().pmoe_fused_moe_bf16_workspace_bytes(M, K, N, sorted_token_ids.numel(),
                                                                                 int(split)), x.device)
            _check(lib().pmoe_fused_moe_bf16_ex(*common, _p(workspace), workspace.numel() * workspace.element_size(),
                                                _p(live_rows), _p(out_rows), _stream()))
        elif workspace is None:
            _check(lib().pmoe_fused_moe_bf16(*common, _stream()))
        else:
            _check(lib().pmoe_fused_moe_bf16_ws(*common, _p(workspace), workspace.numel() * workspace.element_size(),
                                                _stream()))
    return out


def fused_moe_mxfp8(x, x_scales, w, w_scales, w2, w2_scales, sorted_token_ids, expert_ids,
                    num_tokens_post_padded, topk_weights, out, top_k, block_m=128, block_n=64, warp_n=4,
                    stages=4, bpc=1, split=True, workspace=None, live_rows=None):
    M, K = x.shape
    E, N, _ = w.shape
    with torch.cuda.device(x.device):
        common = (_p(x), _p(x_scales), _p(w), _p(w_scales), _p(w2), _p(w2_scales), _p(out), _p(sorted_token_ids),
                  _p(expert_ids), _p(num_tokens_post_padded), _p(topk_weights), top_k, M, K, N, E,
                  sorted_token_ids.numel(), block_m, block_n, warp_n, stages, bpc, int(split))
        if live_rows is not None:
            if workspace is None:
                workspace = _workspace(lib().pmoe_fused_moe_mxfp8_workspace_bytes(M, K, N, sorted_token_ids.numel(),
                                                                                  int(split)), x.device)
            _check(lib().pmoe_fused_moe_mxfp8_ex(*common, _p(workspace), workspace.numel() * workspace.element_size(),
                                                 _p(live_rows), _stream()))
        elif workspace is None:
            _check(lib().pmoe_fused_moe_mxfp8(*common, _stream()))
        else:
            _check(lib().pmoe_fused_moe_mxfp8_ws(*common, _p(workspace),
                                                 workspace.numel() * workspace.element_size(), _stream()))
    return out


def fused_moe_bf16_keep(x, w, w2, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, out, top_k,
                        bpc=1):
    """``fused_moe_bf16`` (split pipeline; ``bpc`` as ``moe_align`` was run) that also returns the gate/up pre-activations
    ``[sorted_num, N]`` for ``fused_moe_bf16_backward(..., gate_up=...)``."""
    M, K = x.shape
    E, N, _ = w.shape
    R = sorted_token_ids.numel()
    gate_up = torch.empty(R, N, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        workspace = _workspace(lib().pmoe_fused_moe_bf16_workspace_bytes(M, K, N, R, 1), x.device)
        _check(lib().pmoe_fused_moe_bf16_keep_ws(
            _p(x), _p(w), _p(w2), _p(out), _p(sorted_token_ids), _p(expert_ids), _p(num_tokens_post_padded),
            _p(topk_weights), top_k, M, K, N, E, R, bpc, _p(gate_up), _p(workspace),
            workspace.numel() * workspace.element_size(), _stream()))
    return out, gate_up


def fused_moe_bf16_backward(x, w, w2, d_out, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights,
                            top_k, need_weight_grad=True, workspace=None, gate_up=None, d_w=None, accumulate=False):
    """Gradients of ``fused_moe_bf16`` for ``d_out`` [T, K]: ``(d_x [T, K], d_w [E, N, K], d_w2 [E, K, N/2],
    d_topk_weights fp32 [T, top_k] | None)``, the routing tensors being those of the forward call (block_m = 128).
    ``d_w=(d_w, d_w2)``: bf16 or fp32 tensors to write the weight gradients into, or - with ``accumulate`` - to add
    them to."""
    T, K = x.shape
    E, N, _ = w.shape
    assert d_out.shape == x.shape and d_out.dtype == torch.bfloat16 and d_out.is_contiguous()
    d_x = torch.empty_like(x)
    if d_w is None:
        assert not accumulate
        d_w1, d_w2 = torch.empty_like(w), torch.empty_like(w2)
    else:
        d_w1, d_w2 = d_w
        assert d_w1.shape == w.shape and d_w2.shape == w2.shape and d_w1.dtype == d_w2.dtype
        assert d_w1.is_contiguous() and d_w2.is_contiguous()
    dw_dtype = {torch.float32: 0, torch.bfloat16: 1}[d_w1.dtype]
    d_wt = torch.empty(T, top_k, dtype=torch.float32, device=x.device) if need_weight_grad else None
    with torch.cuda.device(x.device):
        if workspace is None:
            workspace = _workspace(lib().pmoe_fused_moe_bf16_backward_workspace_bytes(
                T, K, N, E, top_k, sorted_token_ids.numel()), x.device)
        _check(lib().pmoe_fused_moe_bf16_backward_ex(
            _p(x), _p(w), _p(w2), _p(d_out), _p(sorted_token_ids), _p(expert_ids), _p(num_tokens_post_padded),
            _p(topk_weights), top_k, T, K, N, E, sorted_token_ids.numel(), _p(d_x), _p(d_w1), _p(d_w2), _p(d_wt),
            _p(gate_up), dw_dtype, int(accumulate), _p(workspace), workspace.numel() * workspace.element_size(),
            _stream()))
    return d_x, d_w1, d_w2, d_wt


def route_topk(logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """``(topk_ids int32 [T, top_k], topk_weights fp32 [T, top_k])`` from router logits ``[T, E]`` (fp32 or bf16)."""
    assert logits.is_cuda and logits.dim() == 2 and logits.is_contiguous()
    dtype = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    T, E = logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    wts = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        _check(lib().pmoe_route_topk(_p(logits), dtype, T, E, top_k, int(renormalize), _p(ids), _p(wts), _stream()))
    return ids, wts


def route_topk_align(logits: torch.Tensor, top_k: int, renormalize: bool = True, block_m: int = 128, bpc: int = 1):
    """Router + moe_align in one call: ``(topk_ids, topk_weights, sorted_token_ids, expert_ids, num_tokens_post_padded)``."""
    assert logits.is_cuda and logits.dim() == 2 and logits.is_contiguous()
    dtype = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    T, E = logits.shape
    n, pad_to = T * top_k, block_m * bpc
    max_padded = (n + E * (pad_to - 1) + pad_to - 1) // pad_to * pad_to
    mk = lambda *shape: torch.empty(*shape, dtype=torch.int32, device=logits.device)
    ids, sorted_ids, expert_ids, npp = mk(T, top_k), mk(max_padded), mk(max_padded // block_m), mk(1)
    wts = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    nbytes = lib().pmoe_moe_align_workspace_bytes(n, E)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=logits.device)
    with torch.cuda.device(logits.device):
        _check(lib().pmoe_route_topk_align(_p(logits), dtype, T, E, top_k, int(renormalize), _p(ids), _p(wts), _p(sorted_ids),
                                           _p(expert_ids), _p(npp), block_m, pad_to, max_padded, max_padded // block_m,
                                           _p(ws), nbytes, _stream()))
    return ids, wts, sorted_ids, expert_ids, npp


def quantize_mx(x: torch.Tensor, row_index: torch.Tensor | None = None):
    """bf16 ``[T, K]`` -> ``(e4m3 [R, K], e8m0 [R, K/32])``; with ``row_index`` int32 ``[R]`` output row r is
    ``x[row_index[r]]`` (gather and quantiser in one pass), else R = T."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    T, K = x.shape
    R = T if row_index is None else row_index.numel()
    q = torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
    sc = torch.empty(R, K // 32, dtype=torch.float8_e8m0fnu, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().pmoe_quantize_mx(_p(x), _p(row_index), T, _p(q), _p(sc), R, K, _stream()))
    return q, sc


def device_status() -> int:
    """Synchronises; returns the first error code recorded by a kernel (0 = none)."""
    st = _i(0)
    rc = lib().pmoe_device_status(C.byref(st))
    if rc not in (0, 4):
        _check(rc)
    return st.value


def reset_device_status() -> None:
    _check(lib().pmoe_reset_device_status())
