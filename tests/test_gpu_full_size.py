"""Full-size workloads: properties that need no full float64 oracle, plus the
oracle on sampled (batch, head) slices.  Needs a B200."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_f64 as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["one_pass_backward", "two_pass_backward"])
def fc(request):
    from machinelearning_b200 import flash_cuda
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    assert flash_cuda.mma_available(), flash_cuda.mma_unavailable_reason()
    before = flash_cuda.FUSED_BACKWARD
    flash_cuda.FUSED_BACKWARD = request.param == "one_pass_backward"
    yield flash_cuda
    flash_cuda.FUSED_BACKWARD = before


def sample_heads(B, H, n, seed=0):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(B)), int(rng.integers(H))) for _ in range(n)]


def check_sampled(fc, B, T, H, D, window, sinks, n_heads, gen_dtype):
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda: torch.randn(B, T, H, D, device="cuda", dtype=gen_dtype, generator=g).bfloat16()
    q, k, v, do = mk(), mk(), mk(), mk()
    scale = 1.0 / math.sqrt(D)
    o, lse = fc.fwd(q, k, v, scale, True, window, sinks)
    dq, dk, dv = fc.bwd(do, q, k, v, o, lse, scale, True, window, sinks)
    torch.cuda.synchronize()
    assert torch.isfinite(o).all() and torch.isfinite(dq).all()
    assert torch.isfinite(dk).all() and torch.isfinite(dv).all()
    for b, h in sample_heads(B, H, n_heads):
        ro, rl, rq, rk, rv = orc.attention_head(q, k, v, do, b, h, scale, window, sinks)
        for got, want, name in ((o[b, :, h], ro, "o"), (dq[b, :, h], rq, "dq"),
                                (dk[b, :, h], rk, "dk"), (dv[b, :, h], rv, "dv")):
            err = np.abs(got.double().cpu().numpy() - want).max() / np.abs(want).max()
            assert err <= 2e-2, (name, b, h, err)
        assert np.abs(lse[b, h].double().cpu().numpy() - rl).max() <= 1e-3
    return q, k, v, do, o, lse, dq, dk, dv


def test_config2_causal_bf16_b32_h12_t1024_d64(fc):
    q, k, v, do, o, lse, dq, dk, dv = check_sampled(fc, 32, 1024, 12, 64, 0, 0, 6, torch.float32)
    # linearity of the backward in dO: bwd(2 dO) == 2 bwd(dO) bit-for-bit (powers of two are exact)
    dq2, dk2, dv2 = fc.bwd(do * 2, q, k, v, o, lse, 0.125, True)
    assert torch.equal(dq2, dq * 2) and torch.equal(dk2, dk * 2) and torch.equal(dv2, dv * 2)
    # the fp32 SIMT kernels share no code with the tensor-core ones
    o_s, lse_s = fc.fwd(q, k, v, 0.125, False)
    assert (o_s.float() - o.float()).abs().max() < 2e-2
    assert (lse_s - lse).abs().max() < 1e-3
    # first query row attends only itself: O[:, 0] == V[:, 0]
    assert torch.equal(o[:, 0], v[:, 0])


def test_config3_sliding_window_bf16_t4096_w256(fc):
    B, T, H, D, W = 16, 4096, 16, 64, 256
    q, k, v, do, o, lse, dq, dk, dv = check_sampled(fc, B, T, H, D, W, 0, 3, torch.bfloat16)
    # locality: perturbing keys/values at positions >= 2048 cannot change outputs before 2048,
    # and outputs at or after 2048 + 255 cannot depend on keys before 2048
    k2, v2 = k.clone(), v.clone()
    k2[:, 2048:] = -k2[:, 2048:]
    v2[:, 2048:] = 0
    o2, _ = fc.fwd(q, k2, v2, 0.125, True, W, 0)
    assert torch.equal(o2[:, :2048], o[:, :2048])
    k3 = k.clone()
    k3[:, :2048] = 0
    o3, _ = fc.fwd(q, k3, v, 0.125, True, W, 0)
    assert torch.equal(o3[:, 2048 + W - 1:], o[:, 2048 + W - 1:])


def test_config5_long_context_bf16_t16384_d128_one_batch_element(fc):
    # B=8 is sharded one batch element per GPU; one GPU's share is B=1
    check_sampled(fc, 1, 16384, 16, 128, 0, 0, 1, torch.bfloat16)
