"""A bounded device wait that runs out, end to end: kernel -> status word -> host (needs a B200).

The reference fails closed: its loader never raises and records why the kernel is off
(``nanolab/flash_cuda.py:91-135``), and the mixer then takes the SDPA branch with one warning
(``nanolab/mixers.py:365-370``).  Here the failure can also come from the device: every wait inside
the tensor-core kernels is bounded, and a wait that runs out records a code and lets the CTA leave.
``nlfa_test_wait_timeout`` makes exactly that happen on purpose -- one CTA waits one millisecond on
a barrier nothing arrives at, gives up and returns; nothing faults, traps or spins without a limit.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SENTINEL = 777.0


def _problem():
    torch.manual_seed(3)
    B, T, H, D = 1, 200, 2, 64
    mk = lambda: torch.randn(B, T, H, D, device="cuda").bfloat16()
    return mk(), mk(), mk(), 1.0 / math.sqrt(D)


def _raw_fwd(lib, L, q, k, v, scale, o, lse):
    B, T, H, D = q.shape
    return lib.nlfa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, T, H, H, D,
                        scale, 0, 0, L.DTYPE_BF16, L.PATH_TENSOR, torch.cuda.current_stream().cuda_stream)


def test_give_up_is_seen_by_the_host_refused_and_cleared():
    from machinelearning_b200 import _lib as L, flash_cuda as fc
    from oracle import attention_f64 as orc
    assert fc.is_available(), fc.unavailable_reason()
    lib = L.load()
    q, k, v, scale = _problem()
    fc.fwd(q, k, v, scale, True)                                 # registers the host copy for this device
    torch.cuda.synchronize()
    assert not fc.device_timed_out() and lib.nlfa_peek_status() == 0

    assert lib.nlfa_test_wait_timeout(1_000_000, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()                                     # the kernel returned by itself
    # the host knows without having asked the device
    assert fc.device_timed_out() and lib.nlfa_peek_status() == L.ERR_DEVICE_TIMEOUT
    assert not fc.is_available() and "bounded wait" in fc.unavailable_reason()
    # launches are refused, in C and in Python, instead of handing back unwritten memory
    o = torch.full_like(q, SENTINEL)
    lse = torch.full((1, 2, 200), SENTINEL, device="cuda")
    assert _raw_fwd(lib, L, q, k, v, scale, o, lse) == L.ERR_DEVICE_TIMEOUT
    torch.cuda.synchronize()
    assert bool((o == SENTINEL).all()) and bool((lse == SENTINEL).all())
    with pytest.raises(RuntimeError, match="bounded wait"):
        fc.fwd(q, k, v, scale, True)
    with pytest.raises(RuntimeError, match="bounded wait"):
        fc.bwd(q, q, k, v, q, lse, scale, True)
    # explicit clear: the raw word names the wait that gave up (0x100 | site 0xee)
    assert fc.reset_device_status() == 0x1ee
    assert fc.is_available() and lib.nlfa_peek_status() == 0
    # and the kernels are right again
    o2, lse2 = fc.fwd(q, k, v, scale, True)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, scale)
    assert np.abs(o2.double().cpu().numpy() - o_ref).max() <= 2e-2 * np.abs(o_ref).max()
    assert np.abs(lse2.double().cpu().numpy() - lse_ref).max() <= 1e-3


def test_without_a_host_copy_later_launches_do_nothing_until_the_word_is_read():
    """A C caller that registered no host copy: the launch after a give-up is accepted but every CTA
    finds the word set and leaves at once (outputs untouched); nlfa_device_status reports and clears."""
    from machinelearning_b200 import _lib as L, flash_cuda as fc
    assert fc.is_available(), fc.unavailable_reason()
    lib = L.load()
    q, k, v, scale = _problem()
    dev = torch.cuda.current_device()
    assert lib.nlfa_set_status_mirror(None) == 0
    try:
        assert lib.nlfa_test_wait_timeout(500_000, None) == 0
        torch.cuda.synchronize()
        assert lib.nlfa_peek_status() == 0                       # nobody told the host
        o = torch.full_like(q, SENTINEL)
        lse = torch.full((1, 2, 200), SENTINEL, device="cuda")
        assert _raw_fwd(lib, L, q, k, v, scale, o, lse) == 0      # accepted ...
        torch.cuda.synchronize()
        assert bool((o == SENTINEL).all())                       # ... and a no-op
        raw = ctypes.c_uint(0)
        assert lib.nlfa_device_status(ctypes.byref(raw)) == L.ERR_DEVICE_TIMEOUT and raw.value == 0x1ee
        assert lib.nlfa_device_status(ctypes.byref(raw)) == 0 and raw.value == 0
        assert _raw_fwd(lib, L, q, k, v, scale, o, lse) == 0
        torch.cuda.synchronize()
        assert bool(torch.isfinite(o.float()).all()) and not bool((o == SENTINEL).any())
    finally:
        word = fc._status_words.get(dev)
        assert lib.nlfa_set_status_mirror(word.data_ptr() if word is not None else None) == 0


def test_hook_refuses_limits_beyond_the_kernels_own():
    from machinelearning_b200 import _lib as L
    lib = L.load()
    assert lib.nlfa_test_wait_timeout(0, None) == 14
    assert lib.nlfa_test_wait_timeout(3_000_000_000, None) == 14
    x = torch.zeros(4, device="cuda")
    assert lib.nlfa_set_status_mirror(x.data_ptr()) == 14        # device memory is not a host copy
