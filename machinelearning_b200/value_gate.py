"""The two elementwise steps around the attention core, one kernel each way.

``value_blend(v, v0, vr_lambda)``
    nanolab's value residual, ``(1 - sigmoid(lambda)) * v + sigmoid(lambda) * v0``
    (``nanolab/mixers.py:294-297``), written directly in the kernel dtype -- in torch
    that is two multiplies and an add in float32 plus ``flash_attn``'s cast.
``head_gate(y, gate_logits)``
    the per-head sigmoid gate on the attention output, ``y * sigmoid(gate)[..., None]``
    (``nanolab/mixers.py:340-342``).

Both are ``autograd.Function`` s over the C entry points of ``csrc/epilogue.cu``.  No CPU
path: ``supports_*`` say whether a call can run; the functions raise otherwise.
"""
from __future__ import annotations

import torch

from . import _lib, flash_cuda

_DTYPE_CODE = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16,
               torch.bfloat16: _lib.DTYPE_BF16}


def _lib_or_raise():
    lib = flash_cuda._load()
    if lib is None:
        raise RuntimeError(f"flash_cuda is unavailable ({flash_cuda.unavailable_reason()})")
    return lib


def _stream(t):
    return flash_cuda._stream_of(t.device.index)


def supports_blend(v: torch.Tensor, v0: torch.Tensor, lam: torch.Tensor) -> bool:
    return (v.is_cuda and v0.is_cuda and lam.is_cuda and v.dtype in _DTYPE_CODE and v0.dtype == v.dtype
            and v.shape == v0.shape and v.numel() % 8 == 0 and lam.numel() == 1)


def supports_gate(y: torch.Tensor, gate: torch.Tensor) -> bool:
    return (y.dim() == 4 and y.is_cuda and gate.is_cuda and y.dtype in _DTYPE_CODE and gate.dtype in _DTYPE_CODE
            and tuple(gate.shape) == tuple(y.shape[:3]) and y.shape[-1] in flash_cuda.SUPPORTED_HEAD_DIMS)


def blend_fwd(v, v0, lam32, out_dtype):
    """The blend through the C ABI: contiguous ``v`` / ``v0`` of one dtype, ``lam32`` one float32 on the device."""
    lib = _lib_or_raise()
    out = torch.empty(v.shape, dtype=out_dtype, device=v.device)
    with flash_cuda._on_device(v.device.index):
        st = lib.nlfa_value_blend_fwd(v.data_ptr(), v0.data_ptr(), _DTYPE_CODE[v.dtype], lam32.data_ptr(),
                                      out.data_ptr(), _DTYPE_CODE[out_dtype], v.numel(), _stream(v))
    _lib.check("nlfa_value_blend_fwd", st)
    return out


def blend_bwd(g, v, v0, lam32):
    """(dv, dv0, dlambda float32 [1])."""
    lib = _lib_or_raise()
    dv, dv0 = torch.empty_like(v), torch.empty_like(v0)
    dlam = torch.empty(1, dtype=torch.float32, device=v.device)
    scratch = torch.empty(lib.nlfa_value_blend_scratch_bytes(), dtype=torch.uint8, device=v.device)
    with flash_cuda._on_device(v.device.index):
        st = lib.nlfa_value_blend_bwd(g.data_ptr(), _DTYPE_CODE[g.dtype], v.data_ptr(), v0.data_ptr(),
                                      _DTYPE_CODE[v.dtype], lam32.data_ptr(), dv.data_ptr(), dv0.data_ptr(),
                                      dlam.data_ptr(), scratch.data_ptr(), scratch.numel(), v.numel(), _stream(v))
    _lib.check("nlfa_value_blend_bwd", st)
    return dv, dv0, dlam


def gate_fwd(y, gate):
    lib = _lib_or_raise()
    out = torch.empty_like(y)
    rows, D = y.numel() // y.shape[-1], y.shape[-1]
    with flash_cuda._on_device(y.device.index):
        st = lib.nlfa_head_gate_fwd(y.data_ptr(), _DTYPE_CODE[y.dtype], gate.data_ptr(), _DTYPE_CODE[gate.dtype],
                                    out.data_ptr(), rows, D, _stream(y))
    _lib.check("nlfa_head_gate_fwd", st)
    return out


def gate_bwd(g, y, gate):
    """(dy, dgate)."""
    lib = _lib_or_raise()
    dy, dgate = torch.empty_like(y), torch.empty_like(gate)
    rows, D = y.numel() // y.shape[-1], y.shape[-1]
    with flash_cuda._on_device(y.device.index):
        st = lib.nlfa_head_gate_bwd(g.data_ptr(), y.data_ptr(), _DTYPE_CODE[y.dtype], gate.data_ptr(),
                                    _DTYPE_CODE[gate.dtype], dy.data_ptr(), dgate.data_ptr(), rows, D, _stream(y))
    _lib.check("nlfa_head_gate_bwd", st)
    return dy, dgate


class _ValueBlendFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v, v0, lam, out_dtype):
        v, v0 = v.contiguous(), v0.contiguous()
        lam32 = lam.detach().to(torch.float32).reshape(1).contiguous()
        ctx.save_for_backward(v, v0, lam32)
        ctx.lam_meta = (lam.dtype, lam.shape)
        return blend_fwd(v, v0, lam32, out_dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        v, v0, lam32 = ctx.saved_tensors
        dv, dv0, dlam = blend_bwd(g.contiguous(), v, v0, lam32)
        dtype, shape = ctx.lam_meta
        return dv, dv0, dlam.to(dtype).reshape(shape), None


class _HeadGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gate):
        y, gate = y.contiguous(), gate.contiguous()
        ctx.save_for_backward(y, gate)
        return gate_fwd(y, gate)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        y, gate = ctx.saved_tensors
        return gate_bwd(g.contiguous().to(y.dtype), y, gate)


def value_blend(v: torch.Tensor, v0: torch.Tensor, lam: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """``(1 - sigmoid(lam)) * v + sigmoid(lam) * v0`` in ``out_dtype`` (default: the autocast dtype
    under CUDA autocast -- what ``flash_attn`` would cast to -- else ``v.dtype``)."""
    if not supports_blend(v, v0, lam):
        raise ValueError(f"value_blend: unsupported inputs {tuple(v.shape)} {v.dtype} / {v0.dtype} on {v.device}")
    if out_dtype is None:
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else v.dtype
    if torch.compiler.is_compiling():
        from . import compile_ops              # registered operators: one graph node instead of a graph break
        return compile_ops.value_blend(v, v0, lam, out_dtype)
    if not (torch.is_grad_enabled() and (v.requires_grad or v0.requires_grad or lam.requires_grad)):
        # nothing to differentiate (inference): the kernel alone, no autograd node
        return blend_fwd(v.contiguous(), v0.contiguous(), lam.detach().to(torch.float32).reshape(1).contiguous(),
                         out_dtype)
    return _ValueBlendFn.apply(v, v0, lam, out_dtype)


def head_gate(y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``y * sigmoid(gate)[..., None]`` for ``y [B,T,H,D]`` and gate logits ``[B,T,H]``."""
    if not supports_gate(y, gate):
        raise ValueError(f"head_gate: unsupported inputs {tuple(y.shape)} {y.dtype}, gate {tuple(gate.shape)} "
                         f"{gate.dtype} on {y.device}")
    if torch.compiler.is_compiling():
        from . import compile_ops
        return compile_ops.head_gate(y, gate)
    if not (torch.is_grad_enabled() and (y.requires_grad or gate.requires_grad)):
        return gate_fwd(y.contiguous(), gate.contiguous())
    return _HeadGateFn.apply(y, gate)


def main() -> int:
    """Self-check against the torch expressions these replace, then kernel timings.

        python -m machinelearning_b200.value_gate [--batch 64 --seq 1024 --heads 12 --head_dim 64 --iters 20]

    Timings call the plain ``*_fwd`` / ``*_bwd`` functions (C entry points, CUDA events, no
    autograd); GB/s counts every operand once and every result once.
    """
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--head_dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    if not flash_cuda.is_available():
        print("unavailable:", flash_cuda.unavailable_reason())
        return 1
    B, T, H, D = a.batch, a.seq, a.heads, a.head_dim
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).bfloat16()
    v, v0, gv, y, gy = (rnd(B, T, H, D) for _ in range(5))
    gate = rnd(B, T, H)
    lam = torch.tensor([0.3], device="cuda")

    vs, v0s, ls = v[:2].clone().requires_grad_(), v0[:2].clone().requires_grad_(), lam.clone().requires_grad_()
    value_blend(vs, v0s, ls, out_dtype=torch.bfloat16).backward(gv[:2])
    vr, v0r, lr = v[:2].clone().requires_grad_(), v0[:2].clone().requires_grad_(), lam.clone().requires_grad_()
    s = torch.sigmoid(lr)
    ((1 - s) * vr + s * v0r).to(torch.bfloat16).backward(gv[:2])
    rel = lambda p, q: ((p.float() - q.float()).abs().max() / q.float().abs().max()).item()
    print(f"value blend vs torch (relative): dv {rel(vs.grad, vr.grad):.2e}  dv0 {rel(v0s.grad, v0r.grad):.2e}  "
          f"dlambda {rel(ls.grad, lr.grad):.2e}")
    ys, gs = y[:2].clone().requires_grad_(), gate[:2].clone().requires_grad_()
    head_gate(ys, gs).backward(gy[:2])
    yr, gr = y[:2].clone().requires_grad_(), gate[:2].clone().requires_grad_()
    (yr * torch.sigmoid(gr).unsqueeze(-1)).backward(gy[:2])
    print(f"head gate vs torch (relative): dy {rel(ys.grad, yr.grad):.2e}  dgate {rel(gs.grad, gr.grad):.2e}")

    def time_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters

    n, rows = B * T * H * D, B * T * H
    for name, fn, nbytes in (
            ("value blend forward", lambda: blend_fwd(v, v0, lam, torch.bfloat16), 6 * n),
            ("value blend backward", lambda: blend_bwd(gv, v, v0, lam), 10 * n),
            ("head gate forward", lambda: gate_fwd(y, gate), 4 * n + 2 * rows),
            ("head gate backward", lambda: gate_bwd(gy, y, gate), 6 * n + 4 * rows)):
        ms = time_ms(fn)
        print(f"[{B},{T},{H},{D}] bf16 {name}: {ms * 1e3:.1f} us = {nbytes / ms / 1e6:.0f} GB/s ({nbytes / 1e6:.1f} MB)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
