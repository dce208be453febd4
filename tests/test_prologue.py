"""The fused q/k prologue (RMSNorm + RoPE + cast): oracle against nanolab's own
float64 results (``tests/golden/qk_prologue.npz``), host-side argument checks of the
C entry points, and -- on the GPU -- the kernels against the oracle."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, bf16_bits_to_f32
from oracle import prologue_f64

FIXTURE = GOLDEN / "qk_prologue.npz"


def cases():
    d = np.load(FIXTURE)
    out = []
    for tag in sorted({k.split("/")[0] for k in d.files}):
        B, T, H, D, norm, rope = (int(v) for v in d[f"{tag}/meta"])
        c = dict(tag=tag, B=B, T=T, H=H, D=D, norm=bool(norm), rope=bool(rope),
                 x=bf16_bits_to_f32(d[f"{tag}/x"]), gy=bf16_bits_to_f32(d[f"{tag}/gy"]),
                 w=bf16_bits_to_f32(d[f"{tag}/w"]), y=d[f"{tag}/y"], dx=d[f"{tag}/dx"])
        c["dw"] = d[f"{tag}/dw"] if norm else None
        c["cos"], c["sin"] = (d[f"{tag}/cos"], d[f"{tag}/sin"]) if rope else (None, None)
        out.append(c)
    return out


CASES = cases()
IDS = [f"{c['tag']}-D{c['D']}-norm{int(c['norm'])}-rope{int(c['rope'])}" for c in CASES]


@pytest.mark.parametrize("c", CASES, ids=IDS)
def test_oracle_matches_nanolab_float64(c):
    w = c["w"] if c["norm"] else None
    y, _ = prologue_f64.forward(c["x"], w, c["cos"], c["sin"])
    dx, dw = prologue_f64.backward(c["gy"], c["x"], w, c["cos"], c["sin"])
    assert np.abs(y - c["y"]).max() <= 1e-12
    assert np.abs(dx - c["dx"]).max() <= 1e-12
    if c["norm"]:
        assert np.abs(dw - c["dw"]).max() <= 1e-11
    if c["rope"]:
        cos, sin = prologue_f64.rope_tables(c["T"], c["D"])
        # float32 arithmetic on both sides: a last-place difference in base**(-2i/D) between numpy and
        # torch is multiplied by the position, hence a bound that grows with T
        tol = 2e-7 * c["T"]
        assert np.abs(cos - c["cos"]).max() <= tol and np.abs(sin - c["sin"]).max() <= tol


def test_entry_points_refuse_bad_arguments_before_any_launch():
    from machinelearning_b200 import _build, _lib
    _build.build()
    lib = _lib.load()
    fwd, bwd = lib.nlfa_qk_prologue_fwd, lib.nlfa_qk_prologue_bwd
    assert lib.nlfa_qk_prologue_scratch_bytes(64) >= 148 * 64 * 4
    ok = (16, 16, None, None, None, 16, 2, None, 1, 4, 2)        # x, dtype, w, cos, sin, y, dtype, rstd, B, T, H
    assert fwd(*ok, 48, 1e-6, None) == 4                          # head dim
    assert fwd(16, 7, None, None, None, 16, 2, None, 1, 4, 2, 64, 1e-6, None) == 3      # dtype
    assert fwd(None, 2, None, None, None, 16, 2, None, 1, 4, 2, 64, 1e-6, None) == 1    # null x
    assert fwd(16, 2, 16, None, None, 16, 2, None, 1, 4, 2, 64, 1e-6, None) == 1        # weight without rstd
    assert fwd(16, 2, None, 16, None, 16, 2, None, 1, 4, 2, 64, 1e-6, None) == 1        # cos without sin
    assert fwd(8, 2, None, None, None, 16, 2, None, 1, 4, 2, 64, 1e-6, None) == 6       # misaligned
    assert fwd(None, 2, None, None, None, None, 2, None, 0, 4, 2, 64, 1e-6, None) == 0  # empty batch
    assert fwd(16, 2, None, None, None, 16, 2, None, -1, 4, 2, 64, 1e-6, None) == 2
    assert bwd(16, 2, 16, 2, 16, None, None, 16, 16, 16, 16, 8, 1, 4, 2, 64, None) == 11   # scratch too small
    assert bwd(None, 2, 16, 2, None, None, None, None, 16, None, None, 0, 1, 4, 2, 64, None) == 1


def test_python_wrapper_rejects_cpu_tensors():
    from machinelearning_b200 import qk_prologue
    x = torch.zeros(1, 4, 2, 64)
    assert not qk_prologue.supports(x, None, None, None)
    with pytest.raises(ValueError):
        qk_prologue.qk_prologue(x)


# ---------------------------------------------------------------- GPU parity
DTYPES = [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16),
          (torch.float16, torch.float16)]


def _rel(a, ref):
    return np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30)


@pytest.mark.gpu
@pytest.mark.parametrize("din,dout", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("c", CASES, ids=IDS)
def test_kernels_match_the_oracle(c, din, dout):
    """fp32 in and out: max-abs 1e-5 (2e-5 on gradients, 1e-4 relative on the weight gradient, a sum
    over every row); 16-bit on either side: 2e-2 relative, ``max|x - ref| / max|ref|``."""
    from machinelearning_b200 import qk_prologue
    dev = "cuda"
    x = torch.from_numpy(c["x"]).to(dev, din).requires_grad_()
    w = torch.from_numpy(c["w"]).to(dev).requires_grad_() if c["norm"] else None
    cos = torch.from_numpy(c["cos"]).to(dev, torch.float32) if c["rope"] else None
    sin = torch.from_numpy(c["sin"]).to(dev, torch.float32) if c["rope"] else None
    gy = torch.from_numpy(c["gy"]).to(dev, dout)
    y = qk_prologue.qk_prologue(x, w, cos, sin, out_dtype=dout)
    assert y.dtype == dout and y.is_contiguous()
    y.backward(gy)
    assert x.grad.dtype == din
    exact = din == torch.float32 and dout == torch.float32
    yn, dxn = y.detach().float().cpu().numpy(), x.grad.float().cpu().numpy()
    if exact:
        assert np.abs(yn - c["y"]).max() <= 1e-5
        assert np.abs(dxn - c["dx"]).max() <= 2e-5
    else:
        assert _rel(yn, c["y"]) <= 2e-2
        assert _rel(dxn, c["dx"]) <= 2e-2
    if c["norm"]:
        assert _rel(w.grad.cpu().numpy(), c["dw"]) <= (1e-4 if exact else 2e-2)


@pytest.mark.gpu
def test_whole_model_size_properties_and_reproducibility():
    """B=8 of the whole-model shape (T=1024, H=12, D=64, bf16): a rotation keeps every row's norm, so with
    a unit weight each output row has squared norm D; the weight gradient is bit-reproducible; rows and
    positions beyond the first are handled like the first (a batch element repeated gives repeated rows)."""
    from machinelearning_b200 import qk_prologue, whole_model
    B, T, H, D = 8, 1024, 12, 64
    g = torch.Generator().manual_seed(5)
    x1 = torch.randn(1, T, H, D, generator=g).bfloat16()
    x = x1.expand(B, T, H, D).contiguous().cuda().requires_grad_()
    w = torch.ones(D, device="cuda", requires_grad=True)
    cos, sin = whole_model.rope_tables(T, D, 10000.0, "cuda", torch.float32)
    y = qk_prologue.qk_prologue(x, w, cos, sin)
    n2 = y.float().pow(2).sum(-1)
    assert (n2 - D).abs().max().item() <= 0.02 * D
    assert torch.equal(y[0], y[B - 1])
    gy = torch.randn(1, T, H, D, generator=g).bfloat16().expand(B, T, H, D).contiguous().cuda()
    y.backward(gy)
    dw1, dx1 = w.grad.clone(), x.grad.clone()
    assert torch.equal(dx1[0], dx1[B - 1])
    w.grad = None
    x.grad = None
    qk_prologue.qk_prologue(x, w, cos, sin).backward(gy)
    assert torch.equal(w.grad, dw1) and torch.equal(x.grad, dx1)
    # against the float64 oracle on a slice (the oracle finishes in seconds at this size)
    ref_y, _ = prologue_f64.forward(x1[:, :64].float().numpy(), np.ones(D), cos[:64].double().cpu().numpy(),
                                    sin[:64].double().cpu().numpy())
    assert _rel(y.detach()[0:1, :64].float().cpu().numpy(), ref_y) <= 2e-2
