"""``torch.library`` registration of the attention kernels, for ``torch.compile``.

nanolab compiles its model when ``Config.compile`` is on (``nanolab/train.py:213-214``).
``flash_cuda.flash_attn`` is an ``autograd.Function`` around ctypes calls, which the
compiler cannot trace: the graph breaks at every layer.  Registered as custom operators
with shape functions and an autograd formula, the same calls become single opaque nodes
of the traced graph, forward and backward.

    from machinelearning_b200 import compile_ops
    y = compile_ops.flash_attn(q, k, v, scale, window=0, sinks=0)      # same contract as flash_cuda.flash_attn

``flash_cuda.flash_attn`` itself takes this route while a compiler is tracing, and so do
``qk_prologue.qk_prologue``, ``value_gate.value_blend`` and ``value_gate.head_gate`` (operators
``nlfa::qk_prologue_*``, ``nlfa::value_blend_*``, ``nlfa::head_gate_*`` below).  The operators
run only the library's kernels; there is no CPU implementation, only the shape functions
tracing needs.
"""
from __future__ import annotations

import math

import torch

from . import flash_cuda


@torch.library.custom_op("nlfa::attn_fwd", mutates_args=(), device_types="cuda")
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, use_mma: bool, window: int,
             sinks: int, block: int) -> tuple[torch.Tensor, torch.Tensor]:
    return flash_cuda.fwd(q, k, v, scale, use_mma, window, sinks, block)


@attn_fwd.register_fake
def _(q, k, v, scale, use_mma, window, sinks, block):
    B, T, H, _ = q.shape
    return torch.empty_like(q), q.new_empty((B, H, T), dtype=torch.float32)


@torch.library.custom_op("nlfa::attn_bwd", mutates_args=(), device_types="cuda")
def attn_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
             lse: torch.Tensor, scale: float, use_mma: bool, window: int,
             sinks: int, block: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return flash_cuda.bwd(dout.contiguous(), q, k, v, o, lse, scale, use_mma, window, sinks, block=block)


@attn_bwd.register_fake
def _(dout, q, k, v, o, lse, scale, use_mma, window, sinks, block):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup(ctx, inputs, output):
    q, k, v, scale, use_mma, window, sinks, block = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse)
    ctx.args = (scale, use_mma, window, sinks, block)


def _backward(ctx, dout, dlse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = attn_bwd(dout, q, k, v, o, lse, *ctx.args)
    return dq, dk, dv, None, None, None, None, None


attn_fwd.register_autograd(_backward, setup_context=_setup)


def flash_attn(q, k, v, scale=None, use_mma=None, *, window: int = 0, sinks: int = 0, block: int = 0):
    """``flash_cuda.flash_attn`` through the registered operators (same checks, same casts)."""
    q, k, v, scale, use_mma = flash_cuda.prepare(q, k, v, scale, use_mma, window, sinks, block)
    return attn_fwd(q, k, v, float(scale), bool(use_mma), int(window), int(sinks), int(block))[0]


# ---------------------------------------------------------------- q/k prologue, value blend, head gate
from typing import Optional  # noqa: E402

from . import qk_prologue as _qp  # noqa: E402
from . import value_gate as _vg  # noqa: E402


@torch.library.custom_op("nlfa::qk_prologue_fwd", mutates_args=(), device_types="cuda")
def qk_prologue_fwd(x: torch.Tensor, weight: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                    sin: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
    return _qp.fwd(x, weight, cos, sin, eps, out_dtype)


@qk_prologue_fwd.register_fake
def _(x, weight, cos, sin, eps, out_dtype):
    rows = x.shape[0] * x.shape[1] * x.shape[2] if weight is not None else 1
    return x.new_empty(x.shape, dtype=out_dtype), x.new_empty((rows,), dtype=torch.float32)


@torch.library.custom_op("nlfa::qk_prologue_bwd", mutates_args=(), device_types="cuda")
def qk_prologue_bwd(gy: torch.Tensor, x: torch.Tensor, weight: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                    sin: Optional[torch.Tensor], rstd: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return _qp.bwd(gy.contiguous(), x, weight, cos, sin, rstd)


@qk_prologue_bwd.register_fake
def _(gy, x, weight, cos, sin, rstd):
    return torch.empty_like(x), x.new_empty((x.shape[-1] if weight is not None else 1,), dtype=torch.float32)


def _qp_setup(ctx, inputs, output):
    x, weight, cos, sin, eps, out_dtype = inputs
    ctx.save_for_backward(x, weight, cos, sin, output[1])
    ctx.has_weight = weight is not None


def _qp_backward(ctx, gy, grstd):
    x, weight, cos, sin, rstd = ctx.saved_tensors
    gx, gw = qk_prologue_bwd(gy, x, weight, cos, sin, rstd)
    return gx, (gw if ctx.has_weight else None), None, None, None, None


qk_prologue_fwd.register_autograd(_qp_backward, setup_context=_qp_setup)


def qk_prologue(x, weight, cos, sin, eps, out_dtype):
    """``qk_prologue.qk_prologue`` through the registered operators (float32 weight and tables)."""
    f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()
    return qk_prologue_fwd(x.contiguous(), f32(weight), f32(cos), f32(sin), float(eps), out_dtype)[0]


@torch.library.custom_op("nlfa::value_blend_fwd", mutates_args=(), device_types="cuda")
def value_blend_fwd(v: torch.Tensor, v0: torch.Tensor, lam: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    return _vg.blend_fwd(v, v0, lam, out_dtype)


@value_blend_fwd.register_fake
def _(v, v0, lam, out_dtype):
    return v.new_empty(v.shape, dtype=out_dtype)


@torch.library.custom_op("nlfa::value_blend_bwd", mutates_args=(), device_types="cuda")
def value_blend_bwd(g: torch.Tensor, v: torch.Tensor, v0: torch.Tensor,
                    lam: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _vg.blend_bwd(g.contiguous(), v, v0, lam)


@value_blend_bwd.register_fake
def _(g, v, v0, lam):
    return torch.empty_like(v), torch.empty_like(v0), lam.new_empty((1,), dtype=torch.float32)


def _vb_setup(ctx, inputs, output):
    v, v0, lam, out_dtype = inputs
    ctx.save_for_backward(v, v0, lam)


def _vb_backward(ctx, g):
    v, v0, lam = ctx.saved_tensors
    dv, dv0, dlam = value_blend_bwd(g, v, v0, lam)
    return dv, dv0, dlam, None


value_blend_fwd.register_autograd(_vb_backward, setup_context=_vb_setup)


def value_blend(v, v0, lam, out_dtype):
    lam32 = lam.to(torch.float32).reshape(1)
    return value_blend_fwd(v.contiguous(), v0.contiguous(), lam32, out_dtype)


@torch.library.custom_op("nlfa::head_gate_fwd", mutates_args=(), device_types="cuda")
def head_gate_fwd(y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    return _vg.gate_fwd(y, gate)


@head_gate_fwd.register_fake
def _(y, gate):
    return torch.empty_like(y)


@torch.library.custom_op("nlfa::head_gate_bwd", mutates_args=(), device_types="cuda")
def head_gate_bwd(g: torch.Tensor, y: torch.Tensor, gate: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return _vg.gate_bwd(g.contiguous().to(y.dtype), y, gate)


@head_gate_bwd.register_fake
def _(g, y, gate):
    return torch.empty_like(y), torch.empty_like(gate)


def _hg_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _hg_backward(ctx, g):
    y, gate = ctx.saved_tensors
    return head_gate_bwd(g, y, gate)


head_gate_fwd.register_autograd(_hg_backward, setup_context=_hg_setup)


def head_gate(y, gate):
    return head_gate_fwd(y.contiguous(), gate.contiguous())
