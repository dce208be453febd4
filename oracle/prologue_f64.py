"""TEST INFRASTRUCTURE -- float64 restatement of the tensor passes nanolab runs on
q and k in front of the attention core.  Never imported by the product path.

Forward, per head row x of D elements at position t:

    y   = x / sqrt(mean(x^2) + eps) * weight          RMSNorm, nanolab/mixers.py:46-56
    out = y * cos[t] + (-y_hi, y_lo) * sin[t]         apply_rope, nanolab/mixers.py:68-75

with cos / sin from ``build_rope_cache`` (``mixers.py:59-65``): angles
t * base^(-2i/D) for i < D/2, repeated for both halves.  ``backward`` is the closed
form of what autograd computes for those lines.  Parity pinned:
``tests/golden/qk_prologue.npz`` was written from nanolab's own ``RMSNorm`` /
``apply_rope`` + autograd in float64 (``tests/golden/make_prologue_golden.py``) and
``tests/test_prologue.py`` holds this file to it at 1e-12.
"""
from __future__ import annotations

import numpy as np


def rope_tables(T: int, D: int, base: float = 10000.0):
    """cos, sin ``[T, D]`` (``build_rope_cache``, ``mixers.py:59-65``).  nanolab forms the
    angles and their cosines in float32 whatever dtype it returns, so the tables are float32
    values here too (returned as float64 arrays)."""
    inv = (np.float32(1.0) / np.power(np.float32(base), np.arange(0, D, 2, dtype=np.float32) / np.float32(D)))
    ang = np.outer(np.arange(T, dtype=np.float32), inv.astype(np.float32)).astype(np.float32)
    ang = np.concatenate([ang, ang], axis=-1)
    return np.cos(ang).astype(np.float64), np.sin(ang).astype(np.float64)


def _rot(y):
    half = y.shape[-1] // 2
    return np.concatenate([-y[..., half:], y[..., :half]], axis=-1)


def _rot_t(g):
    """Transpose of ``_rot``: <rot(y), g> == <y, rot_t(g)>."""
    half = g.shape[-1] // 2
    return np.concatenate([g[..., half:], -g[..., :half]], axis=-1)


def forward(x, weight=None, cos=None, sin=None, eps: float = 1e-6):
    """x ``[B,T,H,D]`` -> (out ``[B,T,H,D]``, rstd ``[B,T,H]``); None skips a stage."""
    x = np.asarray(x, dtype=np.float64)
    rstd = 1.0 / np.sqrt((x * x).mean(-1) + eps)
    y = x * rstd[..., None] * np.asarray(weight, dtype=np.float64) if weight is not None else x
    if cos is not None:
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        y = y * c + _rot(y) * s
    return y, rstd


def backward(g, x, weight=None, cos=None, sin=None, eps: float = 1e-6):
    """Gradient of ``forward``'s output -> (dx ``[B,T,H,D]``, dweight ``[D]`` or None)."""
    g = np.asarray(g, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    if cos is not None:
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        g = g * c + _rot_t(g * s)
    if weight is None:
        return g, None
    w = np.asarray(weight, dtype=np.float64)
    rstd = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    xn = x * rstd
    dweight = (g * xn).reshape(-1, x.shape[-1]).sum(0)
    gw = g * w
    dx = rstd * (gw - xn * (gw * xn).mean(-1, keepdims=True))
    return dx, dweight
