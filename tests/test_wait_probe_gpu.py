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
