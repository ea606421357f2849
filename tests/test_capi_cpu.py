"""Host-side checks that need no GPU: the C ABI library loads, exports every symbol the header declares,
and rejects bad arguments with the documented codes before touching the device; the torch operators are
registered with the reference's schemas."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from prime_flash_moe_b200 import capi
    return capi.lib()


def test_every_declared_symbol_is_exported(lib):
    from prime_flash_moe_b200 import capi
    header = (ROOT / "include" / "pmoe_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(pmoe_\w+)\s*\(", header))
    assert len(declared) >= 13
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/pmoe_b200.h but not exported"
    assert declared == set(capi.SIGNATURES), "capi.SIGNATURES must mirror the header"
    assert lib.pmoe_version() >= 100


def test_moe_align_argument_errors(lib):
    buf = (C.c_int * 4096)()
    p = C.addressof(buf)
    assert lib.pmoe_moe_align(0, p, p, p, 4, 8, 128, 128, 1024, 8, None) == 1          # null pointer
    assert b"null" in lib.pmoe_last_error()
    assert lib.pmoe_moe_align(p, p, p, p, 4, 2000, 128, 128, 1 << 20, 1 << 13, None) == 2  # > 1024 experts
    assert b"1024" in lib.pmoe_last_error()
    assert lib.pmoe_moe_align(p, p, p, p, 4, 8, 128, 128, 128, 1, None) == 1             # max_padded too small
    assert lib.pmoe_moe_align(p, p, p, p, 4, 8, 128, 100, 1024, 8, None) == 1            # pad_to % block_m
    assert lib.pmoe_moe_align_workspace_bytes(1024, 128) == 0                            # single-CTA path
    assert lib.pmoe_moe_align_workspace_bytes(1 << 19, 128) > 0


def _bf16_call(lib, **kw):
    a = dict(top_k=2, M=8, K=256, N=512, E=4, sorted_num=512, block_m=128, block_n=64, warp_n=4, stages=2, bpc=1,
             cpc=1, split=0)
    a.update(kw)
    buf = (C.c_char * 4096)()
    p = (C.addressof(buf) + 1023) & ~1023
    return lib.pmoe_fused_moe_bf16(p, p, p, p, p, p, p, p, a["top_k"], a["M"], a["K"], a["N"], a["E"],
                                   a["sorted_num"], a["block_m"], a["block_n"], a["warp_n"], a["stages"], a["bpc"],
                                   a["cpc"], a["split"], None)


def test_fused_bf16_argument_errors(lib):
    """Same rejections as the reference's TORCH_CHECKs (prime_moe/csrc/torch_interface.cpp:132-139)."""
    assert _bf16_call(lib, K=200) == 1 and b"multiple of 128" in lib.pmoe_last_error()
    assert _bf16_call(lib, N=384) == 1
    assert _bf16_call(lib, block_n=64, warp_n=8) == 2
    assert _bf16_call(lib, stages=6) == 2
    assert _bf16_call(lib, stages=5, split=1) == 2 and b"stages<=4" in lib.pmoe_last_error()
    assert _bf16_call(lib, block_m=64) == 2 and b"block_m=128" in lib.pmoe_last_error()
    assert _bf16_call(lib, cpc=2) == 2
    assert _bf16_call(lib, bpc=3) == 2
    assert _bf16_call(lib, bpc=2, split=0) == 2 and b"split=True" in lib.pmoe_last_error()
    assert _bf16_call(lib, bpc=2, split=1, sorted_num=384) == 1     # tables must be padded to 256 rows
    assert _bf16_call(lib, M=0) == 1
    assert lib.pmoe_fused_moe_bf16_workspace_bytes(8, 256, 512, 512, 0) >= 8 * 256 * 4   # fp32 split-K buffer
    assert lib.pmoe_fused_moe_bf16_workspace_bytes(8, 256, 512, 512, 1) >= 512 * 256 * 2


@pytest.mark.parametrize("pregather", [None, "0", "1"])
@pytest.mark.parametrize("agather", [None, "tma4", "pre", "lsu"])
@pytest.mark.parametrize("tails", [None, "0"])
@pytest.mark.parametrize("bpc", [1, 2])
def test_bf16_workspace_covers_every_launch_path(lib, monkeypatch, pregather, agather, tails, bpc):
    """The bytes the bf16 launcher touches (row-gathered copy of x, activation, pair / tail lists) never exceed
    the size `pmoe_fused_moe_bf16_workspace_bytes` reports, whatever PMOE_PREGATHER / PMOE_AGATHER /
    PMOE_PAIR_TAILS select at call time (all three are read per call); the reported size depends on none of them."""
    for name, val in (("PMOE_PREGATHER", pregather), ("PMOE_AGATHER", agather), ("PMOE_PAIR_TAILS", tails)):
        if val is None:
            monkeypatch.delenv(name, raising=False)
        else:
            monkeypatch.setenv(name, val)
    shapes = [(4096, 4096, 28672, 8, 2, 10240), (8192, 2048, 1536, 128, 8, 81920), (8, 256, 512, 4, 2, 512),
              (256, 4096, 512, 8, 4, 2048)]
    for M, K, N, E, k, sorted_num in shapes:
        for split in (0, 1):
            if bpc == 2 and not split:
                continue
            size = lib.pmoe_fused_moe_bf16_workspace_bytes(M, K, N, sorted_num, split)
            touched = lib.pmoe_debug_bf16_workspace_extent(M, K, N, E, k, sorted_num, bpc, split)
            assert 0 < touched <= size, (M, K, N, sorted_num, split, bpc, touched, size)
            if split:
                assert size >= sorted_num * (N // 2 + K) * 2 + (sorted_num // 128 + 2) * 4


def test_bf16_ws_entry_point_rejects_a_short_workspace(lib):
    """The `_ws` entry point checks the caller's size against the full layout before any launch."""
    buf = (C.c_char * 8192)()
    p = (C.addressof(buf) + 1023) & ~1023
    need = lib.pmoe_fused_moe_bf16_workspace_bytes(8, 256, 512, 512, 1)
    rc = lib.pmoe_fused_moe_bf16_ws(p, p, p, p, p, p, p, p, 2, 8, 256, 512, 4, 512, 128, 64, 4, 2, 2, 1, 1, p, need - 1,
                                    None)
    assert rc == 1 and str(need).encode() in lib.pmoe_last_error()


def test_backward_argument_errors_and_workspace_plan(lib):
    """The backward entry point validates before it touches the device; its workspace plan covers the row-space
    buffers (xs, d_out rows, gate|up, d_gate|d_up, weighted activation) and grows with every dimension."""
    buf = (C.c_char * 8192)()
    p = (C.addressof(buf) + 1023) & ~1023
    common = (p, p, p, p, p, p, p, p)
    assert lib.pmoe_fused_moe_bf16_backward(*common, 2, 8, 96, 512, 4, 512, p, p, p, None, None, p, 1 << 30, None) == 2
    assert b"multiple of 64" in lib.pmoe_last_error()
    assert lib.pmoe_fused_moe_bf16_backward(*common, 2, 8, 256, 512, 4, 500, p, p, p, None, None, p, 1 << 30, None) == 1
    assert b"sorted_num" in lib.pmoe_last_error()
    assert lib.pmoe_fused_moe_bf16_backward(*common, 2, 8, 256, 512, 2000, 512, p, p, p, None, None, p, 1 << 30,
                                            None) == 2
    assert b"1024 experts" in lib.pmoe_last_error()
    assert lib.pmoe_fused_moe_bf16_backward(None, p, p, p, p, p, p, p, 2, 8, 256, 512, 4, 512, p, p, p, None, None, p,
                                            1 << 30, None) == 1
    need = lib.pmoe_fused_moe_bf16_backward_workspace_bytes(8, 256, 512, 4, 2, 512)
    rows = 512 * (2 * 256 + 2 * 512 + 256) * 2                      # bf16 row-space buffers
    assert need >= rows and need % 1024 == 0
    assert lib.pmoe_fused_moe_bf16_backward(*common, 2, 8, 256, 512, 4, 512, p, p, p, None, None, p, need - 1, None) == 1
    assert str(need).encode() in lib.pmoe_last_error()
    assert lib.pmoe_fused_moe_bf16_backward_workspace_bytes(8, 256, 512, 4, 2, 1024) > need
    assert lib.pmoe_fused_moe_bf16_backward_workspace_bytes(8, 512, 512, 4, 2, 512) > need
    assert lib.pmoe_fused_moe_bf16_keep_ws(*common, 2, 8, 256, 512, 4, 512, 1, None, p, 1 << 30, None) == 1
    assert b"gate_up" in lib.pmoe_last_error()
    assert lib.pmoe_debug_set_backward_mask(127) == 127


def test_wait_limit_argument_range(lib):
    assert lib.pmoe_debug_set_wait_ns(10) == 1                   # below 1 microsecond
    assert lib.pmoe_debug_set_wait_ns(10 ** 12) == 1             # above 60 seconds


def test_operator_schemas_match_reference():
    import prime_flash_moe_b200  # noqa: F401  (registers the ops)
    s = str(torch.ops.prime_moe.fused_moe_bf16.default._schema)
    assert s == ("prime_moe::fused_moe_bf16(Tensor x, Tensor w, Tensor w2, Tensor sorted_token_ids, "
                 "Tensor expert_ids, Tensor num_tokens_post_padded, Tensor topk_weights, Tensor(a!) out, "
                 "int top_k, int block_m, int block_n, int warp_n, int stages, int bpc, int cpc, "
                 "bool split=True) -> ()")
    s = str(torch.ops.prime_moe.fused_moe_mxfp8.default._schema)
    assert s == ("prime_moe::fused_moe_mxfp8(Tensor x, Tensor x_scales, Tensor w, Tensor w_scales, Tensor w2, "
                 "Tensor w2_scales, Tensor sorted_token_ids, Tensor expert_ids, Tensor num_tokens_post_padded, "
                 "Tensor topk_weights, Tensor(a!) out, int top_k, int block_m, int block_n, int warp_n, "
                 "int stages, int bpc, bool split=True) -> ()")
    s = str(torch.ops.prime_moe.moe_align.default._schema)
    assert s == ("prime_moe::moe_align(Tensor topk_ids, int num_experts, int block_m, int bpc) -> "
                 "(Tensor, Tensor, Tensor)")


def test_drop_in_package_surface():
    import prime_moe
    assert set(prime_moe.__all__) >= {"fused_moe_bf16", "fused_moe_mxfp8", "pack_scales_blocked", "BLOCK"}
    assert prime_moe.BLOCK == 32


def test_fake_kernels_and_no_cpu_fallback():
    import prime_flash_moe_b200 as P
    ids = torch.zeros((10, 4), dtype=torch.int32, device="meta")
    s, e, n = P.moe_align(ids, 8, 128, 2)
    assert s.shape == (1024 + 1024,) or s.shape[0] % 256 == 0
    assert e.shape[0] == s.shape[0] // 128 and n.shape == (1,)
    # the operators exist for CUDA tensors only: there is no CPU path to fall back to
    with pytest.raises((NotImplementedError, RuntimeError)):
        P.moe_align(torch.zeros((4, 2), dtype=torch.int32), 8, 128, 1)


def test_pack_scales_blocked_matches_oracle(golden):
    import prime_flash_moe_b200 as P
    from oracle import moe_oracle as O
    for case in golden["pack"]:
        u = case["scales"].view(torch.float8_e8m0fnu)
        assert torch.equal(P.pack_scales_blocked(u).view(torch.uint8), case["packed"])
    u = torch.randint(0, 255, (2, 3, 256, 12), dtype=torch.uint8)
    assert torch.equal(P.pack_scales_blocked(u.view(torch.float8_e8m0fnu)).view(torch.uint8),
                       O.pack_scales_blocked(u.view(torch.float8_e8m0fnu)).view(torch.uint8))
    with pytest.raises(AssertionError):
        P.pack_scales_blocked(torch.zeros(100, 4, dtype=torch.uint8))
