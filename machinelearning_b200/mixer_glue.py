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
"""
from __future__ import annotations

import logging
import sys

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
