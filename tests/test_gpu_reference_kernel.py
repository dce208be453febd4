"""These kernels against the reference's own CUDA kernel on the same GPU.

``oracle/build_ref.py`` compiles ``nanolab/csrc/flash_attn_cuda.cu`` where it lies into
``oracle/_ref/nanolab_flash_attn.so`` (a built file that travels with the repository; the
source does not).  Where that file is absent the tests skip.  The reference kernel is
plain-causal only, so windows are not compared here (the float64 oracle covers them)."""
import json
import math

import numpy as np
import pytest
import torch

from oracle import build_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/nanolab_flash_attn.so was not built (python oracle/build_ref.py)")
    return mod


def _inputs(B, T, H, Hkv, D, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(B, T, h, D, device="cuda", generator=g).to(dtype)
    return mk(H), mk(Hkv), mk(Hkv), mk(H)


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30)).item()


# shapes of the reference's own device tests (nanolab/tests.py:366-372, :443-449) and a C2 slice
SHAPES = [(2, 100, 4, 2, 32), (1, 37, 2, 2, 32), (1, 64, 4, 1, 64), (1, 200, 2, 2, 64), (1, 80, 2, 1, 128),
          (2, 1024, 12, 12, 64)]


@pytest.mark.parametrize("B,T,H,Hkv,D", SHAPES)
@pytest.mark.parametrize("dtype,use_mma", [(torch.float32, False), (torch.bfloat16, True), (torch.float16, True)],
                         ids=["fp32-fma", "bf16-mma", "fp16-mma"])
def test_outputs_and_gradients_match_the_reference_kernel(ref, B, T, H, Hkv, D, dtype, use_mma):
    """fp32: max-abs 1e-5 (O, LSE) and 3e-5 (gradients) -- two fp32-accumulating kernels with different
    summation orders; 16-bit: 2e-2 relative (``max|a - b| / max|b|``), LSE 1e-3 absolute."""
    from machinelearning_b200 import flash_cuda
    q, k, v, do = _inputs(B, T, H, Hkv, D, dtype)
    scale = 1.0 / math.sqrt(D)
    ref_mma = use_mma and D <= 64                                 # the reference has no tensor-core backward at D=128
    o_r, l_r = ref.fwd(q, k, v, scale, ref_mma)
    dq_r, dk_r, dv_r = ref.bwd(do, q, k, v, o_r, l_r, scale, ref_mma)
    o, lse = flash_cuda.fwd(q, k, v, scale, use_mma)
    dq, dk, dv = flash_cuda.bwd(do, q, k, v, o, lse, scale, use_mma)
    if dtype == torch.float32:
        assert (o - o_r).abs().max().item() <= 1e-5 and (lse - l_r).abs().max().item() <= 1e-5
        for a, b in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
            assert (a - b).abs().max().item() <= 3e-5
    else:
        assert _rel(o, o_r) <= 2e-2 and (lse - l_r).abs().max().item() <= 1e-3
        for a, b in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
            assert _rel(a, b) <= 2e-2


def _time(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def test_faster_than_the_reference_kernel_at_the_124m_shape(ref):
    """B=32 H=12 T=1024 D=64 bf16, forward + backward, CUDA events: the reference's tensor-core
    (``mma.sync``) kernels recompiled for this GPU are the baseline to beat."""
    from machinelearning_b200 import flash_cuda
    q, k, v, do = _inputs(32, 1024, 12, 12, 64, torch.bfloat16)
    scale = 0.125
    o_r, l_r = ref.fwd(q, k, v, scale, True)
    o, lse = flash_cuda.fwd(q, k, v, scale, True)
    t_ref = (_time(lambda: ref.fwd(q, k, v, scale, True)), _time(lambda: ref.bwd(do, q, k, v, o_r, l_r, scale, True)))
    t_own = (_time(lambda: flash_cuda.fwd(q, k, v, scale, True)),
             _time(lambda: flash_cuda.bwd(do, q, k, v, o, lse, scale, True)))
    flops = 14.0 * 64 * (1024 * 1025 / 2) * 32 * 12
    line = {"shape": "B=32 H=12 T=1024 D=64 bf16 causal", "reference_kernel_ms": {"fwd": t_ref[0], "bwd": t_ref[1]},
            "these_kernels_ms": {"fwd": t_own[0], "bwd": t_own[1]},
            "reference_tflops": flops / sum(t_ref) / 1e9, "these_tflops": flops / sum(t_own) / 1e9,
            "speedup": sum(t_ref) / sum(t_own)}
    print("\nreference kernel comparison:", json.dumps(line))       # shown with pytest -s
    assert sum(t_own) < sum(t_ref)
