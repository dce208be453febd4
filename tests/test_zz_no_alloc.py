"""The scratch-free backward entry point against the ordinary one (needs a B200).

`nlfa_bwd_static_scratch` exists for callers that cannot hand the library a
scratch buffer -- their device memory is already committed elsewhere, or they
may not call anything that allocates.  It keeps the Delta tape in a fixed array
inside the library, so consecutive calls reuse the same memory; this test makes
two calls in a row, with different upstream gradients, and holds each to the
result of `nlfa_bwd` on the same inputs.  Both entry points run the same
kernels on the same inputs and the kernels are bit-reproducible, so the results
must be equal bit for bit.  It is collected last on purpose, and passes both
alone in a fresh process and after the rest of the suite.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_bwd(lib, L, dout, q, k, v, o, lse, scale, window, sinks, path):
    B, T, H, D = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    code = {torch.float32: L.DTYPE_F32, torch.float16: L.DTYPE_F16, torch.bfloat16: L.DTYPE_BF16}[q.dtype]
    st = lib.nlfa_bwd_static_scratch(
        dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, H, k.shape[2], D, scale, window, sinks,
        code, path, torch.cuda.current_stream().cuda_stream)
    assert st == 0, L.strerror(st)
    return dq, dk, dv


# (B, T, H, Hkv, D, dtype, tensor cores, window, sinks)
CASES = {
    "bf16_gqa": (2, 300, 4, 2, 64, torch.bfloat16, True, 0, 0),
    "bf16_window_with_sinks": (2, 300, 4, 2, 64, torch.bfloat16, True, 96, 4),
    "fp32_simt": (2, 100, 4, 2, 32, torch.float32, False, 0, 0),
    "at_the_limit_1048576_rows": (64, 1024, 16, 16, 32, torch.bfloat16, True, 0, 0),
}


@pytest.mark.parametrize("case", list(CASES))
def test_static_scratch_backward_equals_nlfa_bwd_twice_in_a_row(case):
    from machinelearning_b200 import _lib as L, flash_cuda as fc
    assert fc.is_available(), fc.unavailable_reason()
    assert fc.mma_available(), fc.mma_unavailable_reason()
    lib = L.load()
    B, T, H, Hkv, D, dtype, tensor, window, sinks = CASES[case]
    assert B * H * T <= lib.nlfa_static_scratch_max_rows()
    if case.startswith("at_the_limit"):
        assert B * H * T == lib.nlfa_static_scratch_max_rows()
    scale = 1.0 / math.sqrt(D)
    torch.manual_seed(7)
    mk = lambda h: torch.randn(B, T, h, D, device="cuda").to(dtype)
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    o, lse = fc.fwd(q, k, v, scale, tensor, window, sinks)
    path = L.PATH_TENSOR if tensor else L.PATH_SIMT
    for call in range(2):
        dout = mk(H) * (1.0 + call)                       # second call: other gradients, larger
        want = fc.bwd(dout, q, k, v, o, lse, scale, tensor, window, sinks)   # the existing entry point
        got = _static_bwd(lib, L, dout, q, k, v, o, lse, scale, window, sinks, path)
        torch.cuda.synchronize()
        for name, g, w in zip(("dq", "dk", "dv"), got, want):
            assert torch.isfinite(g.float()).all(), (call, name)
            assert torch.equal(g, w), (call, name, float((g.float() - w.float()).abs().max()))


def test_static_scratch_refuses_problems_beyond_its_limit():
    from machinelearning_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    rows = lib.nlfa_static_scratch_max_rows()
    st = lib.nlfa_bwd_static_scratch(p, p, p, p, p, p, p, p, p, 1, rows + 1, 1, 1, 64, 0.125,
                                     0, 0, _lib.DTYPE_BF16, _lib.PATH_TENSOR, None)
    assert st == 13 and b"1048576" in lib.nlfa_strerror(st)
