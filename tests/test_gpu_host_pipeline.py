"""Host-resident batches through the sliced, stream-overlapped pipeline: results
must be bit-identical to one whole-batch call (batch elements are independent)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pinned(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype).pin_memory()


@pytest.mark.parametrize("B,T,H,Hkv,D,window,sinks,slices", [
    (8, 256, 4, 4, 64, 0, 0, 4),
    (5, 200, 4, 2, 64, 64, 4, 3),      # ragged slices, GQA, window with sinks, odd T
    (2, 384, 2, 2, 128, 0, 0, 8),      # more slices asked for than batch elements
])
def test_pipeline_matches_whole_batch(B, T, H, Hkv, D, window, sinks, slices):
    from machinelearning_b200 import flash_cuda, host_pipeline
    if not flash_cuda.is_available():
        pytest.fail(f"flash_cuda unavailable on a GPU box: {flash_cuda.unavailable_reason()}")
    dev = torch.device("cuda:0")
    dt = torch.bfloat16
    q, do = _pinned((B, T, H, D), 1, dt), _pinned((B, T, H, D), 4, dt)
    k, v = _pinned((B, T, Hkv, D), 2, dt), _pinned((B, T, Hkv, D), 3, dt)
    out = [torch.full_like(t, float("nan")).pin_memory() for t in (q, q, k, v)]
    pipe = host_pipeline.HostPipeline(tuple(q.shape), tuple(k.shape), dt, dev, n_slices=slices)
    scale = 1.0 / math.sqrt(D)
    for _ in range(2):                  # the second call exercises buffer reuse across calls
        pipe.run(q, k, v, do, *out, scale=scale, window=window, sinks=sinks)
    torch.cuda.synchronize()

    qd, kd, vd = (t.to(dev).requires_grad_() for t in (q, k, v))
    y = flash_cuda.flash_attn(qd, kd, vd, scale, use_mma=True, window=window, sinks=sinks)
    grads = torch.autograd.grad(y, (qd, kd, vd), do.to(dev))
    for got, ref in zip(out, (y.detach(), *grads)):
        assert torch.equal(got, ref.cpu())


def test_pipeline_rejects_pageable_memory():
    from machinelearning_b200 import host_pipeline
    dev = torch.device("cuda:0")
    t = torch.zeros(2, 128, 2, 64, dtype=torch.bfloat16)
    pipe = host_pipeline.HostPipeline(tuple(t.shape), tuple(t.shape), t.dtype, dev, n_slices=2)
    with pytest.raises(ValueError):
        pipe.run(t, t, t, t, t, t, t, t)
