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


class _QkPrologueFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cos, sin, eps, out_dtype):
        lib = flash_cuda._load()
        if lib is None:
            raise RuntimeError(f"flash_cuda is unavailable ({flash_cuda.unavailable_reason()})")
        x = x.contiguous()
        B, T, H, D = x.shape
        w, c, s = _f32(weight), _f32(cos), _f32(sin)
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        rstd = torch.empty(B * T * H if w is not None else 1, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            st = lib.nlfa_qk_prologue_fwd(x.data_ptr(), _DTYPE_CODE[x.dtype], _ptr(w), _ptr(c), _ptr(s),
                                          y.data_ptr(), _DTYPE_CODE[out_dtype], rstd.data_ptr(),
                                          B, T, H, D, float(eps), torch.cuda.current_stream().cuda_stream)
        _lib.check("nlfa_qk_prologue_fwd", st)
        ctx.save_for_backward(x, w, c, s, rstd)
        ctx.weight_dtype = None if weight is None else weight.dtype
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy):
        lib = flash_cuda._load()
        x, w, c, s, rstd = ctx.saved_tensors
        gy = gy.contiguous()
        B, T, H, D = x.shape
        gx = torch.empty_like(x)
        gw = torch.empty(D, dtype=torch.float32, device=x.device) if w is not None else None
        nbytes = lib.nlfa_qk_prologue_scratch_bytes(D) if w is not None else 0
        scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=x.device)
        with torch.cuda.device(x.device):
            st = lib.nlfa_qk_prologue_bwd(gy.data_ptr(), _DTYPE_CODE[gy.dtype], x.data_ptr(),
                                          _DTYPE_CODE[x.dtype], _ptr(w), _ptr(c), _ptr(s), rstd.data_ptr(),
                                          gx.data_ptr(), _ptr(gw), scratch.data_ptr(), scratch.numel(),
                                          B, T, H, D, torch.cuda.current_stream().cuda_stream)
        _lib.check("nlfa_qk_prologue_bwd", st)
        if gw is not None and ctx.weight_dtype != torch.float32:
            gw = gw.to(ctx.weight_dtype)
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
    return _QkPrologueFn.apply(x, weight, cos, sin, eps, out_dtype)
