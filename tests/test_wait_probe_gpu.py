"""One bounded wait is made to run out, on purpose and harmlessly: a one-CTA probe kernel waits on an mbarrier
that nothing arrives on, with the wait limit lowered to a few milliseconds. The kernel must end by itself
through its normal exit, leave its code in the device status word (the library then reports PMOE_ERR_DEVICE),
and after `pmoe_reset_device_status` a normal call must work again. No GEMM kernel, no trap, no fault is
involved: this is the same `mbar_wait` every kernel of the library uses, run against a barrier with no
producer."""
import ctypes as C
import time

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DEFAULT_NS = 2_000_000_000


def test_expired_wait_sets_status_and_reset_clears_it():
    from prime_flash_moe_b200 import capi
    lib = capi.lib()
    torch.cuda.set_device(0)
    assert capi.device_status() == 0
    assert lib.pmoe_debug_set_wait_ns(5_000_000) == 0            # 5 ms
    try:
        t0 = time.perf_counter()
        assert lib.pmoe_debug_wait_probe(torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.004 <= waited < 1.0, f"the probe should give up after ~5 ms, took {waited:.4f} s"
        st = C.c_int(0)
        assert lib.pmoe_device_status(C.byref(st)) == 4          # PMOE_ERR_DEVICE
        assert st.value == 9                                     # ST_TIMEOUT_PROBE
        assert b"bounded wait" in lib.pmoe_last_error()
        assert capi.device_status() == 9                         # sticky until reset
    finally:
        capi.reset_device_status()
        assert lib.pmoe_debug_set_wait_ns(DEFAULT_NS) == 0
    assert capi.device_status() == 0
    # the context is intact and a normal call runs to the right result
    x, w1, w2, ids, wts = O.make_case(64, 256, 4, 256, 2, seed=2)
    s, e, n = capi.moe_align(ids.to(DEV), 4, 128, 1)
    out = torch.empty(64, 256, dtype=torch.bfloat16, device=DEV)
    capi.fused_moe_bf16(x.to(DEV), w1.to(DEV), w2.to(DEV), s, e, n, wts.to(DEV), out, 2)
    torch.cuda.synchronize()
    assert O.max_rel_to_peak(out.cpu(), O.moe_ref_fp32(x, w1, w2, ids, wts)) <= 2e-2
    assert capi.device_status() == 0


def test_expert_parallel_flag_wait_runs_out_without_a_peer():
    """The flag waits of the peer-memory exchange, on one GPU: a combine for step 1 of a two-rank group whose second
    rank does not exist - nothing ever sets its flag. With the limit at 5 ms the kernel gives up, records status 12
    (return flags), ends normally, and the library reports it; after the reset a step whose flags ARE set works."""
    from prime_flash_moe_b200 import capi
    lib = capi.lib()
    torch.cuda.set_device(0)
    assert capi.device_status() == 0
    T, K, world = 64, 256, 2
    hdr = lib.pmoe_ep_header_bytes()
    y_off = (hdr + 1023) // 1024 * 1024
    nbytes = y_off + T * world * K * 2
    ptr, handle = C.c_void_p(), C.create_string_buffer(64)
    assert lib.pmoe_ep_buffer_alloc(nbytes, C.byref(ptr), handle) == 0, lib.pmoe_last_error()
    try:
        slot_of = torch.full((T, world), -1, dtype=torch.int32, device=DEV)
        slot_of[:, 0] = torch.arange(T, dtype=torch.int32, device=DEV)
        out = torch.full((T, K), float("nan"), dtype=torch.bfloat16, device=DEV)
        stream = torch.cuda.current_stream().cuda_stream
        assert lib.pmoe_debug_set_wait_ns(5_000_000) == 0
        t0 = time.perf_counter()
        assert lib.pmoe_ep_combine_peer(ptr, y_off, slot_of.data_ptr(), out.data_ptr(), T, world, K, 1, stream) == 0
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 2.0
        assert capi.device_status() == 12                      # ST_TIMEOUT_EP_RETURN
        capi.reset_device_status()
        # now publish the flags of both "ranks" for step 1 by hand (header: cnt | disp | comb flags of 32 ints each)
        view = torch.as_tensor(ep_bytes(ptr.value, nbytes), device=DEV)
        flags = view[:3 * 32 * 4].view(torch.int32)
        flags[64] = 1
        flags[65] = 1
        rows = view[y_off:y_off + T * K * 2].view(torch.bfloat16).view(T, K)
        rows.copy_(torch.arange(T, device=DEV, dtype=torch.float32).view(T, 1).expand(T, K).to(torch.bfloat16))
        assert lib.pmoe_ep_combine_peer(ptr, y_off, slot_of.data_ptr(), out.data_ptr(), T, world, K, 1, stream) == 0
        torch.cuda.synchronize()
        assert capi.device_status() == 0
        assert torch.equal(out, rows)
        del view, flags, rows
    finally:
        capi.reset_device_status()
        assert lib.pmoe_debug_set_wait_ns(DEFAULT_NS) == 0
        torch.cuda.synchronize()
        lib.pmoe_ep_buffer_free(ptr)


def ep_bytes(ptr, nbytes):
    from prime_flash_moe_b200.ep import _DeviceBytes
    return _DeviceBytes(ptr, nbytes)
