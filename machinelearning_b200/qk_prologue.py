"""Fused prologue of the attention core: QK-RMSNorm + RoPE + cast, one pass each way.

In nanolab's mixer the attention core is preceded, for q and for k, by
``q_norm`` / ``k_norm`` (``nanolab/mixers.py:287-289``), ``apply_rope``
(``:290-292``) and the cast to the kernel dtype inside ``flash_attn``
(``nanolab/flash_cuda.py:263-266``): about a dozen elementwise kernels forward and
as many backward, each a full pass over ``[B,T,H,D]``.  ``qk_prologue`` does the
same arithmetic in one kernel (``csrc/prologue.cu``) and hands the attention
kernels a tensor that is already in their dtype and contiguous.

    q = qk_prologue(q_proj(x).view(B, T, H, D), q_norm.weight, cos, sin)   # bf16 under autocast
    k = qk_prologue(k_proj(x).view(B, T, Hkv, D), k_norm.weight, cos, sin)
    y = flash_cuda.flash_attn(q, k, v, scale)

No CPU path: ``supports`` says whether a call can run, and ``qk_prologue`` raises
when the library is unavailable.
"""
from __future__ import annotations

import torch

from . import _lib, flash_cuda

_DTYPE_CODE = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16,
               torch.bfloat16: _lib.DTYPE_BF16}
EPS = 1e-6          # nanolab's RMSNorm default (mixers.py:50)


def supports(x: torch.Tensor, weight, cos, sin) -> bool:
    """Pure shape / dtype / device check (no library load), like ``flash_cuda.supports``."""
    if x.dim() != 4 or not x.is_cuda or x.dtype not in _DTYPE_CODE:
        return False
    D = x.shape[-1]
    if D not in flash_cuda.SUPPORTED_HEAD_DIMS:
        return False
    if weight is not None and (not weight.is_cuda or tuple(weight.shape) != (D,)):
        return False
    if (cos is None) != (sin is None):
        return False
    if cos is not None:
        want = (x.shape[1], D)
        if not cos.is_cuda or tuple(cos.shape) != want or tuple(sin.shape) != want:
            return False
    return True


def _f32(t):
    return None if t is None else t.detach().to(torch.float32).contiguous()


def _ptr(t):
    return None if t is None else t.data_ptr()


def fwd(x, weight, cos, sin, eps: float, out_dtype):
    """(y, rstd) through the C ABI: contiguous CUDA ``x``; float32 ``weight`` / ``cos`` / ``sin`` or None."""
    lib = flash_cuda._load()
    if lib is None:
        raise RuntimeError(f"flash_cuda is unavailable ({flash_cuda.unavailable_reason()})")
    B, T, H, D = x.shape
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    rstd = torch.empty(B * T * H if weight is not None else 1, dtype=torch.float32, device=x.device)
    index = x.device.index
    with flash_cuda._on_device(index):
        st = lib.nlfa_qk_prologue_fwd(x.data_ptr(), _DTYPE_CODE[x.dtype], _ptr(weight), _ptr(cos), _ptr(sin),
                                      y.data_ptr(), _DTYPE_CODE[out_dtype], rstd.data_ptr(),
                                      B, T, H, D, float(eps), flash_cuda._stream_of(index))
    if st:
        _lib.check("nlfa_qk_prologue_fwd", st)
    return y, rstd


def bwd(gy, x, weight, cos, sin, rstd):
    """(gx, gweight) through the C ABI; ``gweight`` is float32 ``[D]`` (a 1-element dummy without a weight)."""
    lib = flash_cuda._load()
    if lib is None:
        raise RuntimeError(f"flash_cuda is unavailable ({flash_cuda.unavailable_reason()})")
    B, T, H, D = x.shape
    gx = torch.empty_like(x)
    gw = torch.empty(D if weight is not None else 1, dtype=torch.float32, device=x.device)
    nbytes = lib.nlfa_qk_prologue_scratch_bytes(D) if weight is not None else 0
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=x.device)
    index = x.device.index
    with flash_cuda._on_device(index):
        st = lib.nlfa_qk_prologue_bwd(gy.data_ptr(), _DTYPE_CODE[gy.dtype], x.data_ptr(), _DTYPE_CODE[x.dtype],
                                      _ptr(weight), _ptr(cos), _ptr(sin), rstd.data_ptr(), gx.data_ptr(),
                                      gw.data_ptr() if weight is not None else None, scratch.data_ptr(),
                                      scratch.numel(), B, T, H, D, flash_cuda._stream_of(index))
    if st:
        _lib.check("nlfa_qk_prologue_bwd", st)
    return gx, gw


class _QkPrologueFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cos, sin, eps, out_dtype):
        x = x.contiguous()
        w, c, s = _f32(weight), _f32(cos), _f32(sin)
        y, rstd = fwd(x, w, c, s, eps, out_dtype)
        ctx.save_for_backward(x, w, c, s, rstd)
        ctx.weight_dtype = None if weight is None else weight.dtype
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy):
        x, w, c, s, rstd = ctx.saved_tensors
        gx, gw = bwd(gy.contiguous(), x, w, c, s, rstd)
        gw = None if w is None else gw.to(ctx.weight_dtype)
        return gx, gw, None, None, None, None


def qk_prologue(x: torch.Tensor, weight=None, cos=None, sin=None, eps: float = EPS, out_dtype=None):
    """``cast(rope(rms_norm(x) * weight))`` on ``[B,T,H,D]``; ``None`` skips a stage.

    ``out_dtype`` defaults to what ``flash_attn`` would cast to: the autocast dtype
    when CUDA autocast is on (``nanolab/flash_cuda.py:161-177``), else ``x.dtype``.
    Raises ``ValueError`` for inputs ``supports`` rejects.
    """
    if not supports(x, weight, cos, sin):
        raise ValueError(f"qk_prologue: unsupported inputs {tuple(x.shape)} {x.dtype} on {x.device}")
    if out_dtype is None:
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
    if out_dtype not in _DTYPE_CODE:
        raise ValueError(f"qk_prologue: unsupported output dtype {out_dtype}")
    if torch.compiler.is_compiling():
        from . import compile_ops              # registered operators: one graph node instead of a graph break
        return compile_ops.qk_prologue(x, weight, cos, sin, eps, out_dtype)
    if not (torch.is_grad_enabled() and (x.requires_grad or (weight is not None and weight.requires_grad))):
        # nothing to differentiate (inference): the kernel alone, no autograd node
        return fwd(x.contiguous(), _f32(weight), _f32(cos), _f32(sin), eps, out_dtype)[0]
    return _QkPrologueFn.apply(x, weight, cos, sin, eps, out_dtype)


def _time_ms(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def main() -> int:
    """Self-check against the torch passes this replaces, then timings of the two kernels.

        python -m machinelearning_b200.qk_prologue [--batch 64 --seq 1024 --heads 12 --head_dim 64 --iters 20]

    Timings call the C entry points on preallocated buffers (CUDA events, no autograd), so
    they are kernel times; GB/s counts one read of x (and gy), one write of y (or gx) and
    the float32 rstd tape.
    """
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--head_dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--in_dtype", default="bf16", choices=("bf16", "fp32"))
    a = ap.parse_args()
    if not flash_cuda.is_available():
        print("unavailable:", flash_cuda.unavailable_reason())
        return 1
    lib = flash_cuda._load()
    B, T, H, D = a.batch, a.seq, a.heads, a.head_dim
    din = torch.bfloat16 if a.in_dtype == "bf16" else torch.float32
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(B, T, H, D, device="cuda", generator=g).to(din)
    gy = torch.randn(B, T, H, D, device="cuda", generator=g).bfloat16()
    w = 1 + 0.1 * torch.randn(D, device="cuda", generator=g)
    half = torch.arange(0, D, 2, device="cuda").float() / D
    ang = torch.outer(torch.arange(T, device="cuda").float(), 10000.0 ** -half)
    ang = torch.cat((ang, ang), dim=-1)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    # correctness: the separate torch passes on a slice
    xs = x[:2].clone().requires_grad_()
    ws = w.clone().requires_grad_()
    y = qk_prologue(xs, ws, cos, sin, out_dtype=torch.bfloat16)
    y.backward(gy[:2])
    xr = x[:2].clone().requires_grad_()
    wr = w.clone().requires_grad_()
    n = torch.nn.functional.rms_norm(xr, (D,), wr, EPS)
    lo, hi = n.chunk(2, dim=-1)
    yr = (n * cos[None, :, None, :] + torch.cat((-hi, lo), dim=-1) * sin[None, :, None, :]).to(torch.bfloat16)
    yr.backward(gy[:2])
    rel = lambda p, q: ((p.float() - q.float()).abs().max() / q.float().abs().max()).item()
    print(f"vs torch passes (relative to the largest magnitude): y {rel(y, yr):.2e}  dx {rel(xs.grad, xr.grad):.2e}  "
          f"dweight {rel(ws.grad, wr.grad):.2e}")

    out = torch.empty(B, T, H, D, device="cuda", dtype=torch.bfloat16)
    gx = torch.empty_like(x)
    rstd = torch.empty(B * T * H, device="cuda", dtype=torch.float32)
    gw = torch.empty(D, device="cuda", dtype=torch.float32)
    scratch = torch.empty(lib.nlfa_qk_prologue_scratch_bytes(D), device="cuda", dtype=torch.uint8)
    st = torch.cuda.current_stream().cuda_stream
    cx, cg = _DTYPE_CODE[din], _lib.DTYPE_BF16

    def fwd():
        _lib.check("fwd", lib.nlfa_qk_prologue_fwd(x.data_ptr(), cx, w.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                                  out.data_ptr(), cg, rstd.data_ptr(), B, T, H, D, EPS, st))

    def bwd():
        _lib.check("bwd", lib.nlfa_qk_prologue_bwd(gy.data_ptr(), cg, x.data_ptr(), cx, w.data_ptr(), cos.data_ptr(),
                                                  sin.data_ptr(), rstd.data_ptr(), gx.data_ptr(), gw.data_ptr(),
                                                  scratch.data_ptr(), scratch.numel(), B, T, H, D, st))
    n_el, es = B * T * H * D, x.element_size()
    tf, tb = _time_ms(fwd, a.iters), _time_ms(bwd, a.iters)
    fb, bb = n_el * (es + 2) + 4 * B * T * H, n_el * (2 + 2 * es) + 4 * B * T * H
    print(f"[{B},{T},{H},{D}] {a.in_dtype} -> bf16: forward {tf * 1e3:.1f} us = {fb / tf / 1e6:.0f} GB/s ({fb / 1e6:.1f} MB); "
          f"backward {tb * 1e3:.1f} us = {bb / tb / 1e6:.0f} GB/s ({bb / 1e6:.1f} MB)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
