"""ctypes loader for ``oracle/_ref/libprime_moe_ref.so`` (the reference's own sm_100a kernels built by
``oracle/build_ref.py``). TEST INFRASTRUCTURE ONLY: used by the GPU parity tests and by the benchmark's
reference-kernel leg; the product never loads it."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libprime_moe_ref.so"
_vp, _i = C.c_void_p, C.c_int
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    global _lib
    if _lib is None:
        h = C.CDLL(str(LIB_PATH))
        h.ref_last_error.restype = C.c_char_p
        h.ref_moe_align.argtypes = [_vp] * 4 + [_i] * 6 + [_vp]
        h.ref_fused_moe_bf16.argtypes = [_vp] * 8 + [_i] * 13 + [_vp]
        h.ref_fused_moe_mxfp8.argtypes = [_vp] * 11 + [_i] * 12 + [_vp]
        _lib = h
    return _lib


def _check(rc):
    if rc:
        raise RuntimeError("reference kernel: " + lib().ref_last_error().decode())


def _s():
    return torch.cuda.current_stream().cuda_stream


def moe_align(topk_ids, num_experts, block_m=128, bpc=1):
    n = topk_ids.numel()
    pad_to = block_m * bpc
    max_padded = (n + num_experts * (pad_to - 1) + pad_to - 1) // pad_to * pad_to
    mk = lambda k: torch.empty(k, dtype=torch.int32, device=topk_ids.device)
    s, e, npp = mk(max_padded), mk(max_padded // block_m), mk(1)
    _check(lib().ref_moe_align(topk_ids.data_ptr(), s.data_ptr(), e.data_ptr(), npp.data_ptr(), n, num_experts,
                               block_m, pad_to, max_padded, max_padded // block_m, _s()))
    return s, e, npp


def fused_moe_bf16(x, w, w2, s, e, npp, tw, out, top_k, block_m=128, block_n=64, warp_n=4, stages=2, bpc=1, cpc=1,
                   split=True):
    M, K = x.shape
    E, N, _ = w.shape
    _check(lib().ref_fused_moe_bf16(x.data_ptr(), w.data_ptr(), w2.data_ptr(), out.data_ptr(), s.data_ptr(),
                                    e.data_ptr(), npp.data_ptr(), tw.data_ptr(), top_k, M, K, N, E, s.numel(),
                                    block_m, block_n, warp_n, stages, bpc, cpc, int(split), _s()))
    return out


def fused_moe_mxfp8(x, xs, w, ws, w2, w2s, s, e, npp, tw, out, top_k, block_m=128, block_n=64, warp_n=4, stages=2,
                    bpc=1, split=True):
    M, K = x.shape
    E, N, _ = w.shape
    _check(lib().ref_fused_moe_mxfp8(x.data_ptr(), xs.data_ptr(), w.data_ptr(), ws.data_ptr(), w2.data_ptr(),
                                     w2s.data_ptr(), out.data_ptr(), s.data_ptr(), e.data_ptr(), npp.data_ptr(),
                                     tw.data_ptr(), top_k, M, K, N, E, s.numel(), block_m, block_n, warp_n, stages,
                                     bpc, int(split), _s()))
    return out
