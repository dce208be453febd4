"""Glue between nanolab's attention mixer and this package's kernels.

Two things a nanolab maintainer needs, as code rather than as a patch in a
document:

``install()``
    makes ``import nanolab.flash_cuda`` (``nanolab/mixers.py:38``) resolve to
    ``machinelearning_b200.flash_cuda``.  Call it before ``nanolab.mixers`` is
    imported; nanolab itself is not modified.

``attention_core(mixer, q, k, v, scale)``
    the routing decision of ``Attention._flash_cuda_attn``
    (``nanolab/mixers.py:347-370``) extended to sliding windows: the reference
    declines every step whose mixer has ``swa_window`` set because its kernel
    takes no mask (``mixers.py:357``); these kernels take ``window`` / ``sinks``
    with the mask of ``sliding_window_mask`` (``mixers.py:125-132``) and ``block``
    with that of ``block_causal_mask`` (``mixers.py:78-93``; a non-causal step is
    one block of the whole sequence), so every mask the mixer has goes through.  Returns the ``[B,T,H,D]``
    result, or ``None`` when the caller should use its SDPA branch -- with the
    reason logged once per mixer, as the reference does, so that an enabled flag
    never silently means nothing.

``fuse_mixer()``
    the other maintainer-side patch as code: it replaces ``nanolab.mixers.Attention.forward``
    (``nanolab/mixers.py:280-345``) by ``fused_attention_forward``, which takes the steps the
    kernels can take -- CUDA tensors, ``flash_cuda=True``, supported shapes -- through one kernel each
    for QK-norm + RoPE + cast (``qk_prologue``), the value-residual blend and the head gate
    (``value_gate``) around the attention core with every mask routed (``attention_core``'s rules),
    and hands every other step to nanolab's own ``forward`` untouched.  At nanolab's 124M shape the
    elementwise passes around the core cost more than the core; the flag alone therefore changes
    little (torch's SDPA is a good kernel too), the fused mixer is what moves tokens/s.
"""
from __future__ import annotations

import importlib
import logging
import sys

import torch

from . import flash_cuda

log = logging.getLogger("machinelearning_b200.mixer_glue")


def install(package: str = "nanolab") -> None:
    """Register this package's ``flash_cuda`` as ``<package>.flash_cuda``.

    Works whether or not ``<package>`` has been imported already, as long as
    ``<package>.mixers`` has not (it binds the module at import time).
    """
    name = f"{package}.flash_cuda"
    if f"{package}.mixers" in sys.modules and sys.modules.get(name) is not flash_cuda:
        raise RuntimeError(f"{package}.mixers is already imported and bound to another flash_cuda")
    sys.modules[name] = flash_cuda
    pkg = sys.modules.get(package)
    if pkg is not None:
        setattr(pkg, "flash_cuda", flash_cuda)


def decline_reason(mixer, q, k, v) -> str | None:
    """Why this step cannot go through the kernels (``None``: it can).

    Pure attribute, shape and dtype checks first; the library is only loaded when
    those pass (the reference orders its checks the same way so that a CPU tensor
    never triggers a build, ``mixers.py:358-361``).
    """
    if not getattr(mixer, "flash_cuda", False):
        return "flash_cuda is off"
    window = int(getattr(mixer, "swa_window", 0) or 0)
    sinks = int(getattr(mixer, "swa_sinks", 0) or 0)
    block = mask_block(mixer, q.shape[1])
    if window and not getattr(mixer, "causal", True):
        return "SWA is causal-only"                                 # the mixer raises for this itself (mixers.py:323-325)
    try:
        flash_cuda.check_window(window, sinks, block)
    except ValueError as e:
        return str(e)
    if not flash_cuda.supports(q, k, v):
        return f"unsupported inputs: {tuple(q.shape)} {q.dtype} on {q.device}"
    if not flash_cuda.is_available():
        return flash_cuda.unavailable_reason()
    return None


def mask_block(mixer, T: int) -> int:
    """The block length of the mixer's current mask, 0 for a causal one: ``block_attn`` when set
    (``nanolab/mixers.py:319-321``), and -- a non-causal step being one bidirectional block -- ``T``
    when ``causal`` is off (``mixers.py:338``, ``is_causal=self.causal``)."""
    block = int(getattr(mixer, "block_attn", 0) or 0)
    if block > 0:
        return block
    return 0 if getattr(mixer, "causal", True) else int(T)


def attention_core(mixer, q, k, v, scale):
    """``[B,T,H,D]`` attention for ``mixer``'s current step, or ``None`` (use SDPA)."""
    why = decline_reason(mixer, q, k, v)
    if why is None:
        return flash_cuda.flash_attn(q, k, v, scale,
                                     window=int(getattr(mixer, "swa_window", 0) or 0),
                                     sinks=int(getattr(mixer, "swa_sinks", 0) or 0),
                                     block=mask_block(mixer, q.shape[1]))
    if getattr(mixer, "flash_cuda", False) and not getattr(mixer, "_flash_declined", False):
        try:
            mixer._flash_declined = True
        except AttributeError:
            pass
        log.warning("flash_cuda=True but the kernel cannot run (%s) -> SDPA", why)
    return None


_PLAIN_FORWARD: dict[type, object] = {}        # mixer class -> the forward it had before fuse_mixer()


def fused_attention_forward(self, x, cos, sin, v0=None):
    """``Attention.forward`` of nanolab (``mixers.py:280-345``) for a step the kernels take: the same
    projections, then one kernel each for QK-norm + RoPE + cast, the value-residual blend
    (``mixers.py:294-297``) and the head gate (``mixers.py:340-342``) around the attention core.  Same
    return value ``(o_proj(y), raw_v)``.  A step the kernels decline -- flag off, CPU tensors, shapes or
    masks they do not take, library not loaded or timed out -- goes to the class's own ``forward``,
    with nanolab's own warnings and errors."""
    from . import qk_prologue, value_gate
    plain = _PLAIN_FORWARD[next(c for c in type(self).__mro__ if c in _PLAIN_FORWARD)]
    if not (getattr(self, "flash_cuda", False) and x.is_cuda):
        return plain(self, x, cos, sin, v0)
    B, T, _ = x.shape
    H, Hkv, D = self.n_head, self.n_kv_head, self.head_dim
    q = self.q_proj(x).view(B, T, H, D)
    k = self.k_proj(x).view(B, T, Hkv, D)
    v = raw_v = self.v_proj(x).view(B, T, Hkv, D)
    if decline_reason(self, q, k, v) is not None:
        return plain(self, x, cos, sin, v0)

    qw = self.q_norm.weight if self.qk_norm else None
    kw = self.k_norm.weight if self.qk_norm else None
    if ((qw is not None or cos is not None) and qk_prologue.supports(q, qw, cos, sin)
            and qk_prologue.supports(k, kw, cos, sin)):
        eps = self.q_norm.eps if self.qk_norm else qk_prologue.EPS
        q = qk_prologue.qk_prologue(q, qw, cos, sin, eps)
        k = qk_prologue.qk_prologue(k, kw, cos, sin, self.k_norm.eps if self.qk_norm else eps)
    else:                                                    # nanolab's own lines (mixers.py:287-292)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        if cos is not None:
            rope = sys.modules[type(self).__module__].apply_rope
            q, k = rope(q, cos, sin), rope(k, cos, sin)

    if self.value_residual and v0 is not None:
        if value_gate.supports_blend(v, v0, self.vr_lambda):
            v = value_gate.value_blend(v, v0, self.vr_lambda)
        else:
            lam = torch.sigmoid(self.vr_lambda)
            v = (1 - lam) * v + lam * v0

    y = flash_cuda.flash_attn(q, k, v, self.attn_scale,
                              window=int(self.swa_window or 0), sinks=int(self.swa_sinks or 0),
                              block=mask_block(self, T))
    if self.gated:
        logits = self.gate(x)
        if value_gate.supports_gate(y, logits):
            y = value_gate.head_gate(y, logits)
        else:
            y = y * torch.sigmoid(logits).unsqueeze(-1)
    return self.o_proj(y.reshape(B, T, H * D)), raw_v


def fuse_mixer(package: str = "nanolab") -> None:
    """Route ``<package>.mixers.Attention.forward`` through ``fused_attention_forward``.  Call after
    ``install()``; imports ``<package>.mixers`` if it is not imported yet.  ``unfuse_mixer`` undoes it."""
    mixers = importlib.import_module(f"{package}.mixers")
    if getattr(mixers, "flash_cuda", None) is not flash_cuda:
        raise RuntimeError(f"{package}.mixers is bound to another flash_cuda; call install() before importing it")
    cls = mixers.Attention
    if cls.forward is fused_attention_forward:
        return
    _PLAIN_FORWARD[cls] = cls.forward
    cls.forward = fused_attention_forward


def unfuse_mixer(package: str = "nanolab") -> None:
    mixers = sys.modules.get(f"{package}.mixers")
    cls = getattr(mixers, "Attention", None)
    if cls is not None and cls in _PLAIN_FORWARD:
        cls.forward = _PLAIN_FORWARD.pop(cls)
