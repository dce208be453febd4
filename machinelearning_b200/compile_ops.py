"""``torch.library`` registration of the attention kernels, for ``torch.compile``.

nanolab compiles its model when ``Config.compile`` is on (``nanolab/train.py:213-214``).
``flash_cuda.flash_attn`` is an ``autograd.Function`` around ctypes calls, which the
compiler cannot trace: the graph breaks at every layer.  Registered as custom operators
with shape functions and an autograd formula, the same calls become single opaque nodes
of the traced graph, forward and backward.

    from machinelearning_b200 import compile_ops
    y = compile_ops.flash_attn(q, k, v, scale, window=0, sinks=0)      # same contract as flash_cuda.flash_attn

``flash_cuda.flash_attn`` itself takes this route while a compiler is tracing.  The
operators run only the library's kernels (they call ``flash_cuda.fwd`` / ``flash_cuda.bwd``);
there is no CPU implementation, only the shape functions tracing needs.
"""
from __future__ import annotations

import math

import torch

from . import flash_cuda


@torch.library.custom_op("nlfa::attn_fwd", mutates_args=(), device_types="cuda")
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, use_mma: bool, window: int,
             sinks: int) -> tuple[torch.Tensor, torch.Tensor]:
    return flash_cuda.fwd(q, k, v, scale, use_mma, window, sinks)


@attn_fwd.register_fake
def _(q, k, v, scale, use_mma, window, sinks):
    B, T, H, _ = q.shape
    return torch.empty_like(q), q.new_empty((B, H, T), dtype=torch.float32)


@torch.library.custom_op("nlfa::attn_bwd", mutates_args=(), device_types="cuda")
def attn_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
             lse: torch.Tensor, scale: float, use_mma: bool, window: int,
             sinks: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return flash_cuda.bwd(dout.contiguous(), q, k, v, o, lse, scale, use_mma, window, sinks)


@attn_bwd.register_fake
def _(dout, q, k, v, o, lse, scale, use_mma, window, sinks):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup(ctx, inputs, output):
    q, k, v, scale, use_mma, window, sinks = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse)
    ctx.args = (scale, use_mma, window, sinks)


def _backward(ctx, dout, dlse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = attn_bwd(dout, q, k, v, o, lse, *ctx.args)
    return dq, dk, dv, None, None, None, None


attn_fwd.register_autograd(_backward, setup_context=_setup)


def flash_attn(q, k, v, scale=None, use_mma=None, *, window: int = 0, sinks: int = 0):
    """``flash_cuda.flash_attn`` through the registered operators (same checks, same casts)."""
    q, k, v, scale, use_mma = flash_cuda.prepare(q, k, v, scale, use_mma, window, sinks)
    return attn_fwd(q, k, v, float(scale), bool(use_mma), int(window), int(sinks))[0]
