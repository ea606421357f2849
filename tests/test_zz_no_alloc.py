"""`pmoe_moe_align_static`: the routing kernel for hosts that cannot allocate device memory.

Servers that freeze their device-memory budget after start-up, or plugins running inside another
framework's allocator hooks, can neither call cudaMalloc nor lend a workspace. This entry point keeps
its scratch in a fixed array inside the library. The test drives it through the C ABI, twice in a row
on different inputs (the array keeps the first call's contents), and requires the three outputs to be
identical, integer for integer, to those of the allocating entry point `pmoe_moe_align` and to the CPU
restatement of the reference's algorithm.

Collected last on purpose: a failure here must not hide the result of any other test.
"""
import ctypes as C

import numpy as np

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(fn, ids, E, block_m=128, bpc=1):
    n = ids.numel()
    pad_to = block_m * bpc
    max_padded = (n + E * (pad_to - 1) + pad_to - 1) // pad_to * pad_to
    max_blocks = max_padded // block_m
    mk = lambda k: torch.full((k,), -7, dtype=torch.int32, device=DEV)
    s, e, npp = mk(max_padded), mk(max_blocks), mk(1)
    rc = fn(ids.data_ptr(), s.data_ptr(), e.data_ptr(), npp.data_ptr(), n, E, block_m, pad_to, max_padded,
            max_blocks, torch.cuda.current_stream().cuda_stream)
    return rc, s, e, npp


def test_static_scratch_matches_allocating_entry_point_twice():
    from prime_flash_moe_b200 import capi
    lib = capi.lib()
    assert lib.pmoe_moe_align_static_capacity_bytes() == 256 << 10
    # two different problems, both large enough to need scratch (n > 4096), run back to back
    problems = [(8192, 128, 8, 1, "uniform", 21), (20000, 64, 4, 2, "zipf", 22), (8192, 128, 8, 1, "uniform", 23)]
    for T, E, k, bpc, dist, seed in problems:
        ids, _ = O.make_routing(T, E, k, seed=seed, dist=dist)
        ids = ids.to(DEV)
        assert lib.pmoe_moe_align_workspace_bytes(ids.numel(), E) > 0
        rc, s, e, npp = _call(lib.pmoe_moe_align_static, ids, E, 128, bpc)
        assert rc == 0, lib.pmoe_last_error().decode()
        rc2, s2, e2, npp2 = _call(lib.pmoe_moe_align, ids, E, 128, bpc)
        assert rc2 == 0, lib.pmoe_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(npp, npp2)
        assert torch.equal(e, e2)
        assert torch.equal(s, s2)
        # and, directly, to the CPU restatement of the reference's algorithm
        want_s, want_e, want_n = O.moe_align_spec(ids.cpu().numpy(), E, 128, bpc)
        assert np.array_equal(s.cpu().numpy(), want_s)
        assert np.array_equal(e.cpu().numpy(), want_e)
        assert np.array_equal(npp.cpu().numpy(), want_n)
    # a small problem takes the single-CTA path and needs no scratch at all
    ids, _ = O.make_routing(100, 16, 4, seed=5)
    ids = ids.to(DEV)
    rc, s, e, npp = _call(lib.pmoe_moe_align_static, ids, 16)
    rc2, s2, e2, npp2 = _call(lib.pmoe_moe_align, ids, 16)
    torch.cuda.synchronize()
    assert rc == 0 and rc2 == 0
    assert torch.equal(s, s2) and torch.equal(e, e2) and torch.equal(npp, npp2)
    assert capi.device_status() == 0


def test_static_entry_point_takes_no_device_memory():
    """What the entry point is for: a call must not take device memory from anywhere. Outputs are allocated first,
    the entry point is warmed up once (its first call per device looks up the array's address), and then the
    driver's free-memory figure and the sizes of torch's pools must be the same before and after more calls."""
    from prime_flash_moe_b200 import capi
    lib = capi.lib()
    T, E, k = 8192, 128, 8
    ids, _ = O.make_routing(T, E, k, seed=31)
    ids = ids.to(DEV)
    n = ids.numel()
    max_padded = (n + E * 127 + 127) // 128 * 128
    s = torch.empty(max_padded, dtype=torch.int32, device=DEV)
    e = torch.empty(max_padded // 128, dtype=torch.int32, device=DEV)
    npp = torch.empty(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    call = lambda: lib.pmoe_moe_align_static(ids.data_ptr(), s.data_ptr(), e.data_ptr(), npp.data_ptr(), n, E, 128, 128,
                                             max_padded, max_padded // 128, stream)
    assert call() == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0, allocated0 = torch.cuda.memory_reserved(), torch.cuda.memory_allocated()
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device free memory changed by {free0 - free1} bytes"
    assert (torch.cuda.memory_reserved(), torch.cuda.memory_allocated()) == (reserved0, allocated0)
    want_s, want_e, want_n = O.moe_align_spec(ids.cpu().numpy(), E, 128, 1)
    assert np.array_equal(s.cpu().numpy(), want_s) and np.array_equal(e.cpu().numpy(), want_e)
    assert int(npp.item()) == int(want_n[0])


def test_static_scratch_rejects_oversized_problems():
    from prime_flash_moe_b200 import capi
    lib = capi.lib()
    T, E, k = 40000, 1024, 8           # 1024 experts x one counter per thread block: more than the 256 KiB array holds
    ids = torch.randint(0, E, (T, k), dtype=torch.int32, device=DEV)
    need = lib.pmoe_moe_align_workspace_bytes(ids.numel(), E)
    assert need > lib.pmoe_moe_align_static_capacity_bytes()
    rc, s, e, npp = _call(lib.pmoe_moe_align_static, ids, E)
    torch.cuda.synchronize()
    assert rc == 2                      # PMOE_ERR_UNSUPPORTED
    msg = lib.pmoe_last_error().decode()
    assert str(need) in msg and "pmoe_moe_align_ws" in msg
    assert int(npp.item()) == -7        # nothing was launched
