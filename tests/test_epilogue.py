"""Value blend and head gate (the elementwise steps around the attention core): the oracle
against torch autograd in float64 on nanolab's expressions, host-side argument checks of
the C entry points, and -- on the GPU -- the kernels against the oracle."""
import numpy as np
import pytest
import torch

from oracle import epilogue_f64


def _inputs(seed, B=2, T=19, H=3, D=64):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g).bfloat16().double()
    return dict(v=r(B, T, H, D), v0=r(B, T, H, D), gv=r(B, T, H, D), lam=torch.tensor([0.37], dtype=torch.float64),
                y=r(B, T, H, D), gate=r(B, T, H), gy=r(B, T, H, D))


@pytest.mark.parametrize("seed", [0, 1])
def test_oracle_matches_autograd_on_nanolabs_expressions(seed):
    d = _inputs(seed)
    v, v0, lam = d["v"].clone().requires_grad_(), d["v0"].clone().requires_grad_(), d["lam"].clone().requires_grad_()
    s = torch.sigmoid(lam)                              # nanolab/mixers.py:295-297
    out = (1 - s) * v + s * v0
    out.backward(d["gv"])
    np_ = lambda t: t.detach().numpy()
    assert np.abs(epilogue_f64.blend_forward(np_(v), np_(v0), 0.37) - np_(out)).max() <= 1e-14
    dv, dv0, dl = epilogue_f64.blend_backward(np_(d["gv"]), np_(v), np_(v0), 0.37)
    assert np.abs(dv - np_(v.grad)).max() <= 1e-14 and np.abs(dv0 - np_(v0.grad)).max() <= 1e-14
    assert abs(dl - lam.grad.item()) <= 1e-11
    y, gate = d["y"].clone().requires_grad_(), d["gate"].clone().requires_grad_()
    out = y * torch.sigmoid(gate).unsqueeze(-1)         # nanolab/mixers.py:341-342
    out.backward(d["gy"])
    assert np.abs(epilogue_f64.gate_forward(np_(y), np_(gate)) - np_(out)).max() <= 1e-14
    dy, dg = epilogue_f64.gate_backward(np_(d["gy"]), np_(y), np_(gate))
    assert np.abs(dy - np_(y.grad)).max() <= 1e-14 and np.abs(dg - np_(gate.grad)).max() <= 1e-12


def test_entry_points_refuse_bad_arguments_before_any_launch():
    from machinelearning_b200 import _build, _lib
    _build.build()
    lib = _lib.load()
    assert lib.nlfa_value_blend_scratch_bytes() >= 148 * 4
    assert lib.nlfa_value_blend_fwd(16, 16, 2, 16, 16, 2, 12, None) == 2          # n not a multiple of 8
    assert lib.nlfa_value_blend_fwd(16, 16, 9, 16, 16, 2, 64, None) == 3
    assert lib.nlfa_value_blend_fwd(None, 16, 2, 16, 16, 2, 64, None) == 1
    assert lib.nlfa_value_blend_fwd(16, 8, 2, 16, 16, 2, 64, None) == 6
    assert lib.nlfa_value_blend_fwd(None, None, 2, None, None, 2, 0, None) == 0   # empty
    assert lib.nlfa_value_blend_bwd(16, 2, 16, 16, 2, 16, 16, 16, 16, 16, 4, 64, None) == 11
    assert lib.nlfa_head_gate_fwd(16, 2, 16, 2, 16, 8, 48, None) == 4
    assert lib.nlfa_head_gate_fwd(16, 2, None, 2, 16, 8, 64, None) == 1
    assert lib.nlfa_head_gate_fwd(None, 2, None, 2, None, 0, 64, None) == 0
    assert lib.nlfa_head_gate_bwd(16, 16, 2, 16, 5, 16, 16, 8, 64, None) == 3
    assert lib.nlfa_head_gate_bwd(16, 16, 2, 16, 2, None, 16, 8, 64, None) == 1


def test_python_wrappers_reject_cpu_tensors():
    from machinelearning_b200 import value_gate
    d = _inputs(0)
    assert not value_gate.supports_blend(d["v"], d["v0"], d["lam"])
    assert not value_gate.supports_gate(d["y"], d["gate"])
    with pytest.raises(ValueError):
        value_gate.value_blend(d["v"], d["v0"], d["lam"])
    with pytest.raises(ValueError):
        value_gate.head_gate(d["y"], d["gate"])


def _rel(a, ref):
    return np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30)


@pytest.mark.gpu
@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("din,dout", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                      (torch.float32, torch.bfloat16), (torch.float16, torch.float16)],
                         ids=lambda d: str(d).split(".")[-1])
def test_value_blend_matches_the_oracle(din, dout, D):
    """fp32: 1e-6 max-abs (1e-5 relative on the scalar's gradient, a sum over every element);
    16-bit on either side: 2e-2 relative, ``max|x - ref| / max|ref|``."""
    from machinelearning_b200 import value_gate
    d = _inputs(3, B=2, T=37, H=3, D=D)
    v = d["v"].to("cuda", din).requires_grad_()
    v0 = d["v0"].to("cuda", din).requires_grad_()
    lam = torch.tensor([0.37], device="cuda", requires_grad=True)
    out = value_gate.value_blend(v, v0, lam, out_dtype=dout)
    assert out.dtype == dout
    out.backward(d["gv"].to("cuda", dout))
    np_ = lambda t: t.detach().double().cpu().numpy()
    ref = epilogue_f64.blend_forward(np_(v), np_(v0), 0.37)
    dv, dv0, dl = epilogue_f64.blend_backward(np_(d["gv"]), np_(v), np_(v0), 0.37)
    if din == dout == torch.float32:
        assert np.abs(np_(out) - ref).max() <= 1e-6
        assert np.abs(np_(v.grad) - dv).max() <= 1e-6 and np.abs(np_(v0.grad) - dv0).max() <= 1e-6
        assert abs(lam.grad.item() - dl) <= 1e-5 * max(1.0, abs(dl))
    else:
        assert _rel(np_(out), ref) <= 2e-2
        assert _rel(np_(v.grad), dv) <= 2e-2 and _rel(np_(v0.grad), dv0) <= 2e-2
        assert abs(lam.grad.item() - dl) <= 2e-2 * max(1.0, abs(dl))


@pytest.mark.gpu
@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("dy,dg", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                   (torch.bfloat16, torch.float32)], ids=lambda d: str(d).split(".")[-1])
def test_head_gate_matches_the_oracle(dy, dg, D):
    from machinelearning_b200 import value_gate
    d = _inputs(4, B=2, T=37, H=3, D=D)
    y = d["y"].to("cuda", dy).requires_grad_()
    gate = d["gate"].to("cuda", dg).requires_grad_()
    out = value_gate.head_gate(y, gate)
    assert out.dtype == dy
    out.backward(d["gy"].to("cuda", dy))
    np_ = lambda t: t.detach().double().cpu().numpy()
    ref = epilogue_f64.gate_forward(np_(y), np_(gate))
    ry, rg = epilogue_f64.gate_backward(np_(d["gy"]), np_(y), np_(gate))
    if dy == dg == torch.float32:
        assert np.abs(np_(out) - ref).max() <= 2e-6
        assert np.abs(np_(y.grad) - ry).max() <= 2e-6 and np.abs(np_(gate.grad) - rg).max() <= 2e-5
    else:
        assert _rel(np_(out), ref) <= 2e-2
        assert _rel(np_(y.grad), ry) <= 2e-2 and _rel(np_(gate.grad), rg) <= 2e-2


@pytest.mark.gpu
def test_whole_model_size_is_reproducible_and_ragged_sizes_are_covered():
    """[16,1024,12,64] bf16: two runs give the same bits (fixed-order reductions); a row count that is not
    a multiple of the rows a warp takes per pass leaves no row unwritten."""
    from machinelearning_b200 import value_gate
    g = torch.Generator(device="cuda").manual_seed(0)
    v = torch.randn(16, 1024, 12, 64, device="cuda", generator=g).bfloat16().requires_grad_()
    v0 = torch.randn(16, 1024, 12, 64, device="cuda", generator=g).bfloat16().requires_grad_()
    lam = torch.tensor([-0.2], device="cuda", requires_grad=True)
    gv = torch.randn(16, 1024, 12, 64, device="cuda", generator=g).bfloat16()
    outs = []
    for _ in range(2):
        for t in (v, v0, lam):
            t.grad = None
        value_gate.value_blend(v, v0, lam).backward(gv)
        outs.append((v.grad.clone(), v0.grad.clone(), lam.grad.clone()))
    assert all(torch.equal(a, b) for a, b in zip(*outs))
    s = torch.sigmoid(lam.detach())
    assert torch.allclose(outs[0][0].float(), ((1 - s) * gv.float()), rtol=1e-2, atol=1e-3)
    y = torch.full((1, 37, 3, 64), float("nan"), device="cuda", dtype=torch.bfloat16)
    y.copy_(torch.randn(1, 37, 3, 64, device="cuda", generator=g))
    gate = torch.randn(1, 37, 3, device="cuda", generator=g).bfloat16()
    out = value_gate.head_gate(y, gate)
    assert torch.isfinite(out.float()).all()
    assert torch.allclose(out.float(), y.float() * torch.sigmoid(gate.float())[..., None], rtol=2e-2, atol=1e-3)
