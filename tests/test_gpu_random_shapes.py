"""Seeded random shapes, windows and head groupings through the C ABI against the float64 oracle.

The fixed cases of ``test_gpu_parity.py`` are chosen by hand; this sweep draws 40 configurations from a
seeded generator (odd lengths, lengths around the 128-row tile edges, windows narrower and wider than a
tile, sinks inside and beyond the first block, every head dim and group size) so that a mask or indexing
case nobody thought of still meets the oracle.  Tolerances as in the fixed cases, with two allowances the
sweep needs: float32 gradients are held to 2e-5 times max(1, max|ref| / 4) (a GQA group of four sums four
heads' gradients, so magnitudes grow with the group), and the relative measure's denominator is floored at
1e-2 (with one visible key per row -- T = 1 or window = 1 -- dQ and dK are exactly zero in the oracle)."""
import math
import random

import numpy as np
import pytest
import torch

from oracle import attention_f64 as orc

pytestmark = pytest.mark.gpu


def _configs(n=40, seed=20261125):
    rng = random.Random(seed)
    out = []
    for i in range(n):
        D = rng.choice([32, 64, 64, 128])
        Hkv = rng.choice([1, 2, 3])
        H = Hkv * rng.choice([1, 2, 4])
        T = rng.choice([1, 2, 31, 127, 128, 129, 255, 256, 257, 300, 383, 385, rng.randint(3, 520)])
        B = rng.choice([1, 2])
        if rng.random() < 0.55:
            window = rng.choice([1, 2, 17, 64, 127, 128, 129, 200, 256, T, T + 5])
            sinks = rng.choice([0, 0, 1, 4, 127, 128, 130])
            sinks = min(sinks, window - 1)
        else:
            window = sinks = 0
        dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16, torch.float32])
        out.append((i, B, T, H, Hkv, D, window, sinks, dtype))
    return out


CONFIGS = _configs()


@pytest.mark.parametrize("i,B,T,H,Hkv,D,window,sinks,dtype", CONFIGS,
                         ids=[f"{c[0]}-B{c[1]}T{c[2]}H{c[3]}kv{c[4]}D{c[5]}w{c[6]}s{c[7]}-{str(c[8])[6:]}" for c in CONFIGS])
def test_random_configuration_matches_the_oracle(i, B, T, H, Hkv, D, window, sinks, dtype):
    from machinelearning_b200 import flash_cuda as fc
    assert fc.is_available(), fc.unavailable_reason()
    g = torch.Generator().manual_seed(9000 + i)
    mk = lambda h: torch.randn(B, T, h, D, generator=g).to(dtype).cuda()
    q, k, v, do = mk(H), mk(Hkv), mk(Hkv), mk(H)
    scale = 1.0 / math.sqrt(D)
    use_mma = dtype != torch.float32
    o, lse = fc.fwd(q, k, v, scale, use_mma, window=window, sinks=sinks)
    dq, dk, dv = fc.bwd(do, q, k, v, o, lse, scale, use_mma, window=window, sinks=sinks)
    o_r, lse_r = orc.attention_fwd(q, k, v, scale, window, sinks)
    gq, gk, gv = orc.attention_bwd(do, q, k, v, scale, window, sinks)
    np_ = lambda t: t.double().cpu().numpy()
    if dtype == torch.float32:
        assert np.abs(np_(o) - o_r).max() <= 1e-5 and np.abs(np_(lse) - lse_r).max() <= 1e-5
        for got, want in ((dq, gq), (dk, gk), (dv, gv)):
            assert np.abs(np_(got) - want).max() <= 2e-5 * max(1.0, np.abs(want).max() / 4)
    else:
        rel = lambda got, want: np.abs(np_(got) - want).max() / max(np.abs(want).max(), 1e-2)
        assert rel(o, o_r) <= 2e-2 and np.abs(np_(lse) - lse_r).max() <= 1e-3
        for got, want in ((dq, gq), (dk, gk), (dv, gv)):
            assert rel(got, want) <= 2e-2
    for t in (o, lse, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
