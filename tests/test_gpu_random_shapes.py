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


def _aux_configs(n=24, seed=977):
    rng = random.Random(seed)
    out = []
    for i in range(n):
        D = rng.choice([32, 64, 128])
        out.append((i, rng.choice([1, 2, 3]), rng.choice([1, 2, 7, 33, 100, 257]), rng.choice([1, 2, 3, 5, 12]), D,
                    rng.choice([torch.float32, torch.bfloat16, torch.float16])))
    return out


AUX = _aux_configs()


@pytest.mark.parametrize("i,B,T,H,D,dtype", AUX, ids=[f"{c[0]}-B{c[1]}T{c[2]}H{c[3]}D{c[4]}-{str(c[5])[6:]}" for c in AUX])
def test_random_prologue_blend_and_gate_match_their_oracles(i, B, T, H, D, dtype):
    """The elementwise kernels either side of the core on drawn shapes (row counts that do not fill a
    warp's row groups, one-row tensors, every head dim): fp32 2e-5 max-abs scaled by the reference's
    magnitude, 16-bit 2e-2 relative with the denominator floored at 1e-2."""
    from machinelearning_b200 import qk_prologue, value_gate
    from oracle import epilogue_f64, prologue_f64
    g = torch.Generator().manual_seed(500 + i)
    r = lambda *s: torch.randn(*s, generator=g).to(dtype).cuda()
    np_ = lambda t: t.detach().double().cpu().numpy()

    def close(got, want):
        err = np.abs(np_(got) - want).max()
        if dtype == torch.float32:
            return err <= 2e-5 * max(1.0, np.abs(want).max())
        return err <= 2e-2 * max(np.abs(want).max(), 1e-2)

    x, gy = r(B, T, H, D).requires_grad_(), r(B, T, H, D)
    w = (1 + 0.2 * torch.randn(D, generator=g)).cuda().requires_grad_()
    cos64, sin64 = prologue_f64.rope_tables(T, D)
    cos, sin = (torch.from_numpy(t).float().cuda() for t in (cos64, sin64))
    y = qk_prologue.qk_prologue(x, w, cos, sin, out_dtype=dtype)
    y.backward(gy)
    ref_y, _ = prologue_f64.forward(np_(x), np_(w), cos64, sin64)
    ref_dx, ref_dw = prologue_f64.backward(np_(gy), np_(x), np_(w), cos64, sin64)
    assert close(y, ref_y) and close(x.grad, ref_dx)
    assert np.abs(np_(w.grad) - ref_dw).max() <= (1e-4 if dtype == torch.float32 else 3e-2) * max(np.abs(ref_dw).max(), 1.0)

    v, v0, gv = r(B, T, H, D).requires_grad_(), r(B, T, H, D).requires_grad_(), r(B, T, H, D)
    lam = torch.tensor([-0.4], device="cuda", requires_grad=True)
    out = value_gate.value_blend(v, v0, lam, out_dtype=dtype)
    out.backward(gv)
    dv, dv0, dl = epilogue_f64.blend_backward(np_(gv), np_(v), np_(v0), -0.4)
    assert close(out, epilogue_f64.blend_forward(np_(v), np_(v0), -0.4)) and close(v.grad, dv) and close(v0.grad, dv0)
    assert abs(lam.grad.item() - dl) <= (1e-4 if dtype == torch.float32 else 3e-2) * max(1.0, abs(dl))

    yy, gate, go = r(B, T, H, D).requires_grad_(), r(B, T, H).requires_grad_(), r(B, T, H, D)
    o = value_gate.head_gate(yy, gate)
    o.backward(go)
    dy, dg = epilogue_f64.gate_backward(np_(go), np_(yy), np_(gate))
    assert close(o, epilogue_f64.gate_forward(np_(yy), np_(gate))) and close(yy.grad, dy) and close(gate.grad, dg)
