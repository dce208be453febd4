"""The scratch-free backward entry point against the ordinary one (needs a B200).

`nlfa_bwd_static_scratch` exists for callers that cannot hand the library a
scratch buffer -- their device memory is already committed elsewhere, or they
may not call anything that allocates.  It keeps the Delta tape in a fixed array
inside the library, so consecutive calls reuse the same memory; this test makes
two calls in a row, with different upstream gradients, and holds each to the
result of `nlfa_bwd` on the same inputs.  It is collected last on purpose, and
passes both alone in a fresh process and after the rest of the suite.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

REL_16BIT = 2e-2        # the suite's tolerance for 16-bit tensors: max|x - ref| / max|ref|


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


def test_static_scratch_backward_matches_nlfa_bwd_twice_in_a_row():
    from machinelearning_b200 import _lib, flash_cuda as fc
    assert fc.is_available(), fc.unavailable_reason()
    assert fc.mma_available(), fc.mma_unavailable_reason()
    lib = _lib.load()
    B, T, H, Hkv, D = 2, 300, 4, 2, 64
    assert B * H * T <= lib.nlfa_static_scratch_max_rows()
    scale = 1.0 / math.sqrt(D)
    torch.manual_seed(7)
    mk = lambda h: torch.randn(B, T, h, D, device="cuda").bfloat16()
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    o, lse = fc.fwd(q, k, v, scale, True)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        dout = mk(H) * (1.0 + call)                       # second call: other gradients, larger
        want = fc.bwd(dout, q, k, v, o, lse, scale, True)  # the existing entry point
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        st = lib.nlfa_bwd_static_scratch(
            dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, H, Hkv, D, scale,
            0, 0, _lib.DTYPE_BF16, _lib.PATH_TENSOR, stream)
        assert st == 0, _lib.strerror(st)
        torch.cuda.synchronize()
        for name, got, ref in zip(("dq", "dk", "dv"), (dq, dk, dv), want):
            assert torch.isfinite(got).all(), (call, name)
            assert rel(got, ref) <= REL_16BIT, (call, name)


def test_static_scratch_refuses_problems_beyond_its_limit():
    from machinelearning_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    rows = lib.nlfa_static_scratch_max_rows()
    st = lib.nlfa_bwd_static_scratch(p, p, p, p, p, p, p, p, p, 1, rows + 1, 1, 1, 64, 0.125,
                                     0, 0, _lib.DTYPE_BF16, _lib.PATH_TENSOR, None)
    assert st == 13 and b"1048576" in lib.nlfa_strerror(st)
