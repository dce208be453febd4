"""The ``torch.library`` registration of the attention kernels: shape functions and the autograd
formula on fake tensors (no GPU), and -- on the GPU -- a compiled caller (``aot_eager``: no code
generation, the operators run the library's kernels) against the eager path."""
import math

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

from machinelearning_b200 import compile_ops  # noqa: F401  (registers the operators)


def test_operators_are_registered_with_schemas():
    fwd = torch.ops.nlfa.attn_fwd.default
    bwd = torch.ops.nlfa.attn_bwd.default
    assert "Tensor q, Tensor k, Tensor v, float scale, bool use_mma, SymInt window, SymInt sinks" in str(fwd._schema)
    assert str(bwd._schema).count("Tensor") >= 9


def test_shape_functions_and_autograd_formula_on_fake_tensors():
    with FakeTensorMode():
        q = torch.empty(2, 100, 8, 64, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        k = torch.empty(2, 100, 2, 64, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        v = torch.empty(2, 100, 2, 64, dtype=torch.bfloat16, device="cuda", requires_grad=True)
        o, lse = torch.ops.nlfa.attn_fwd(q, k, v, 0.125, True, 0, 0, 0)
        assert o.shape == q.shape and o.dtype == torch.bfloat16 and o.device.type == "cuda"
        assert lse.shape == (2, 8, 100) and lse.dtype == torch.float32
        assert o.grad_fn is not None                    # the autograd formula is attached
        # running the engine needs a CUDA context even for fake tensors; the backward operator's
        # shape function is checked directly (the GPU tests run the formula end to end)
        dq, dk, dv = torch.ops.nlfa.attn_bwd(torch.empty_like(o), q.detach(), k.detach(), v.detach(), o.detach(),
                                             lse, 0.125, True, 0, 0, 0)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
        assert dk.dtype == torch.bfloat16


@pytest.mark.gpu
@pytest.mark.parametrize("window,sinks", [(0, 0), (96, 4)])
def test_compiled_caller_matches_eager(window, sinks):
    from machinelearning_b200 import flash_cuda
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    torch.manual_seed(0)
    B, T, H, Hkv, D = 2, 300, 4, 2, 64
    q, k, v = (torch.randn(B, T, h, D, device="cuda", dtype=torch.bfloat16, requires_grad=True) for h in (H, Hkv, Hkv))
    w = torch.randn(H * D, H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    do = torch.randn(B, T, H * D, device="cuda", dtype=torch.bfloat16)

    def layer(q, k, v, w):                       # something either side of the operator, as a mixer has
        y = flash_cuda.flash_attn(q * 1.0, k, v, 1.0 / math.sqrt(D), window=window, sinks=sinks)
        return y.reshape(B, T, H * D) @ w

    eager = layer(q, k, v, w)
    g_eager = torch.autograd.grad(eager, (q, k, v, w), do)
    compiled = torch.compile(layer, backend="aot_eager", fullgraph=True)     # fullgraph: a graph break would raise
    out = compiled(q, k, v, w)
    g_out = torch.autograd.grad(out, (q, k, v, w), do)
    assert torch.equal(out, eager)
    for a, b in zip(g_out, g_eager):
        assert torch.equal(a, b)


@pytest.mark.gpu
def test_caller_compiled_with_inductor_keeps_the_operator_whole():
    """nanolab compiles its model with torch's default backend (``nanolab/train.py:213``).  The
    operators must pass through inductor as opaque nodes (``fullgraph=True``: a graph break would
    raise) and still run the library's kernels; the code inductor generates for the caller's own
    operations either side may round differently from eager, hence a tolerance, not bit-equality."""
    from machinelearning_b200 import flash_cuda
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    torch.manual_seed(0)
    B, T, H, Hkv, D = 2, 256, 4, 2, 64
    q, k, v = (torch.randn(B, T, h, D, device="cuda", dtype=torch.bfloat16, requires_grad=True) for h in (H, Hkv, Hkv))
    w = (torch.randn(H * D, H * D, device="cuda") / 16).bfloat16().requires_grad_()
    do = torch.randn(B, T, H * D, device="cuda", dtype=torch.bfloat16)
    calls = {"n": 0}
    real = flash_cuda.fwd

    def counted(*a, **kw):
        calls["n"] += 1
        return real(*a, **kw)

    def layer(q, k, v, w):
        y = flash_cuda.flash_attn(torch.nn.functional.silu(q) + q, k, v, 1.0 / math.sqrt(D), window=96, sinks=4)
        return torch.nn.functional.gelu(y.reshape(B, T, H * D) @ w)

    eager = layer(q, k, v, w)
    g_eager = torch.autograd.grad(eager, (q, k, v, w), do)
    flash_cuda.fwd = counted
    try:
        compiled = torch.compile(layer, backend="inductor", fullgraph=True)
        out = compiled(q, k, v, w)
        g_out = torch.autograd.grad(out, (q, k, v, w), do)
    finally:
        flash_cuda.fwd = real
    assert calls["n"] == 1                        # the compiled graph ran the library's forward
    rel = lambda a, b: float((a.detach().float() - b.detach().float()).abs().max() / b.detach().float().abs().max())
    assert rel(out, eager) <= 2e-2
    for a, b in zip(g_out, g_eager):
        assert rel(a, b) <= 2e-2


def test_prologue_and_epilogue_operators_have_shape_functions():
    with FakeTensorMode():
        x = torch.empty(2, 50, 4, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(64, device="cuda")
        cos = torch.empty(50, 64, device="cuda")
        y, rstd = torch.ops.nlfa.qk_prologue_fwd(x, w, cos, cos, 1e-6, torch.bfloat16)
        assert y.shape == x.shape and y.dtype == torch.bfloat16 and rstd.shape == (400,)
        y32, r1 = torch.ops.nlfa.qk_prologue_fwd(x, None, cos, cos, 1e-6, torch.float32)
        assert y32.dtype == torch.float32 and r1.shape == (1,)
        gx, gw = torch.ops.nlfa.qk_prologue_bwd(y, x, w, cos, cos, rstd)
        assert gx.shape == x.shape and gx.dtype == x.dtype and gw.shape == (64,)
        lam = torch.empty(1, device="cuda")
        out = torch.ops.nlfa.value_blend_fwd(x, x, lam, torch.bfloat16)
        dv, dv0, dl = torch.ops.nlfa.value_blend_bwd(out, x, x, lam)
        assert out.shape == x.shape and dv.shape == x.shape and dl.shape == (1,)
        gate = torch.empty(2, 50, 4, dtype=torch.bfloat16, device="cuda")
        o = torch.ops.nlfa.head_gate_fwd(x, gate)
        dy, dg = torch.ops.nlfa.head_gate_bwd(o, x, gate)
        assert o.shape == x.shape and dy.shape == x.shape and dg.shape == gate.shape and dg.dtype == gate.dtype


@pytest.mark.gpu
def test_compiled_mixer_with_every_fused_step_matches_eager():
    """The whole-model caller's attention mixer (prologue, value blend, core, gate) compiled with
    ``fullgraph=True`` under bf16 autocast: the output equals the eager run bit for bit; gradients agree
    to 1e-2 relative (the traced backward adds the four projections' contributions to ``x.grad`` in another
    order than the eager engine, in bf16)."""
    from machinelearning_b200 import flash_cuda, whole_model as wm
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    torch.manual_seed(0)
    shape = wm.ModelShape(n_layer=1, d_model=256, n_head=4, n_kv_head=2, head_dim=64, block_size=128, vocab_size=64,
                          flash_cuda=True, zero_init_proj=False)
    mixer = wm.Attention(shape).cuda()
    with torch.no_grad():
        mixer.gate.weight.normal_(0.0, 0.05)
        mixer.vr_lambda.fill_(0.3)
    x = torch.randn(2, 128, 256, device="cuda", requires_grad=True)
    v0 = torch.randn(2, 128, 2, 64, device="cuda", dtype=torch.bfloat16)
    cos, sin = wm.rope_tables(128, 64, 10000.0, "cuda", torch.float32)
    go = torch.randn(2, 128, 256, device="cuda", dtype=torch.bfloat16)

    def run(fn):
        for p in mixer.parameters():
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y, _ = fn(x, cos, sin, v0)
        grads = torch.autograd.grad(y, [x, *mixer.parameters()], go)
        return y, grads

    y_e, g_e = run(mixer)
    y_c, g_c = run(torch.compile(mixer, backend="aot_eager", fullgraph=True))
    assert torch.equal(y_e, y_c)
    for a, b in zip(g_e, g_c):
        assert (a.float() - b.float()).abs().max().item() <= 1e-2 * a.float().abs().max().item() + 1e-6


@pytest.mark.gpu
def test_opcheck_passes_on_the_forward_operator():
    from machinelearning_b200 import flash_cuda
    assert flash_cuda.is_available()
    q, k, v = (torch.randn(1, 64, h, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True) for h in (2, 1, 1))
    torch.library.opcheck(torch.ops.nlfa.attn_fwd.default, (q, k, v, 0.125, True, 0, 0, 0),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
