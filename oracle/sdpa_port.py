"""The reference's CPU attention path, restated -- TEST INFRASTRUCTURE.

This is what nanolab runs when the CUDA kernel is not used, and therefore what
the benchmark times on the host cores as the CPU baseline:

* ``sdpa_attention``  -- ``nanolab/flash_cuda.py:282-294`` (``sdpa_reference``) and
  the plain-causal branch of ``Attention.forward`` (``nanolab/mixers.py:310-338``):
  widen KV heads, transpose to [B,H,T,D], ``F.scaled_dot_product_attention``.
* ``swa_attention``   -- the sliding-window branch of the same method
  (``mixers.py:321-335``): ``swa_auto_chunk`` (``:138-165``) picks a chunk, then
  either ``swa_chunked`` (``:168-200``) or the dense ``sliding_window_mask``
  (``:96-135``) goes to SDPA.

The arithmetic is torch's; nothing here is used by the shipped GPU path.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _widen(q, k, v):
    group = q.shape[2] // k.shape[2]
    qs = q.transpose(1, 2)
    ks = k.repeat_interleave(group, dim=2).transpose(1, 2)
    vs = v.repeat_interleave(group, dim=2).transpose(1, 2)
    return qs, ks, vs


def sdpa_attention(q, k, v, scale):
    """Plain causal attention on [B,T,H,D] / [B,T,Hkv,D] through SDPA."""
    qs, ks, vs = _widen(q, k, v)
    y = F.scaled_dot_product_attention(qs, ks, vs, is_causal=True, scale=scale)
    return y.transpose(1, 2).contiguous()


def auto_chunk(T: int, window: int) -> int:
    """Chunk when ``T >= 4*window`` at ``max(256, window)``, else 0 = dense mask."""
    if window <= 0 or T <= 0 or T < 4 * window:
        return 0
    return max(256, window)


def dense_window_mask(T: int, window: int, sinks: int, device) -> torch.Tensor:
    i = torch.arange(T, device=device)
    qpos, kpos = i[:, None], i[None, :]
    causal = kpos <= qpos
    keep = causal & (kpos > qpos - (window - sinks))
    if sinks:
        keep = keep | (causal & (kpos < sinks))
    return keep[None, None]


def chunked_window_attention(qs, ks, vs, window, sinks, scale, chunk):
    """[B,H,T,D] in and out; each query chunk only sees the keys it can reach."""
    B, H, T, D = qs.shape
    span = window - sinks
    out = qs.new_empty(B, H, T, D)
    pos = torch.arange(T, device=qs.device)
    for s0 in range(0, T, chunk):
        e0 = min(s0 + chunk, T)
        lo = max(0, s0 - span + 1)
        if lo <= sinks:
            kc, vc, kpos = ks[:, :, :e0], vs[:, :, :e0], pos[:e0]
        else:
            kc = torch.cat([ks[:, :, :sinks], ks[:, :, lo:e0]], dim=2)
            vc = torch.cat([vs[:, :, :sinks], vs[:, :, lo:e0]], dim=2)
            kpos = torch.cat([pos[:sinks], pos[lo:e0]])
        qpos = pos[s0:e0]
        m = ((kpos[None, :] <= qpos[:, None])
             & ((kpos[None, :] > qpos[:, None] - span) | (kpos[None, :] < sinks)))
        out[:, :, s0:e0] = F.scaled_dot_product_attention(
            qs[:, :, s0:e0], kc, vc, attn_mask=m[None, None], scale=scale)
    return out


def swa_attention(q, k, v, scale, window: int, sinks: int, chunk: int = -1):
    """Sliding-window attention the way the mixer's SDPA branch computes it."""
    qs, ks, vs = _widen(q, k, v)
    T = qs.shape[2]
    c = auto_chunk(T, window) if chunk < 0 else chunk
    if c:
        y = chunked_window_attention(qs, ks, vs, window, sinks, scale, c)
    else:
        mask = dense_window_mask(T, window, sinks, qs.device)
        y = F.scaled_dot_product_attention(qs, ks, vs, attn_mask=mask, scale=scale)
    return y.transpose(1, 2).contiguous()


def cpu_attention(q, k, v, scale, window: int = 0, sinks: int = 0):
    if window:
        return swa_attention(q, k, v, scale, window, sinks)
    return sdpa_attention(q, k, v, scale)


def cpu_fwd_bwd(q, k, v, dout, scale, window: int = 0, sinks: int = 0):
    """Forward + autograd backward on CPU; returns (O, dQ, dK, dV)."""
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    y = cpu_attention(q, k, v, scale, window, sinks)
    dq, dk, dv = torch.autograd.grad(y, (q, k, v), dout)
    return y.detach(), dq, dk, dv
