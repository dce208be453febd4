"""TEST INFRASTRUCTURE -- float64 restatement of the two elementwise steps nanolab's
mixer wraps around the attention core.  Never imported by the product path.

* value blend, ``nanolab/mixers.py:294-297``:
  ``lam = sigmoid(vr_lambda); v = (1 - lam) * v + lam * v0``
* head gate, ``nanolab/mixers.py:340-342``:
  ``g = sigmoid(gate(x)).unsqueeze(-1); y = y * g``

each with the closed form of what autograd computes for it.  nanolab has these as lines
inside ``Attention.forward``, not as functions, so they are pinned two ways:
``tests/test_epilogue.py`` checks this file against torch autograd in float64 on the same
expressions, and ``tests/golden/whole_model_tiny.npz`` (nanolab's own GPT, which contains
both steps in every layer) pins the kernels end to end through ``tests/test_whole_model.py``.
"""
from __future__ import annotations

import numpy as np


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-np.asarray(x, dtype=np.float64)))


def blend_forward(v, v0, lam):
    s = _sigmoid(lam)
    return (1.0 - s) * np.asarray(v, np.float64) + s * np.asarray(v0, np.float64)


def blend_backward(g, v, v0, lam):
    """-> (dv, dv0, dlambda)."""
    g, v, v0 = (np.asarray(t, np.float64) for t in (g, v, v0))
    s = _sigmoid(lam)
    return (1.0 - s) * g, s * g, float((g * (v0 - v)).sum() * s * (1.0 - s))


def gate_forward(y, gate):
    """y ``[..., H, D]``, gate ``[..., H]``."""
    return np.asarray(y, np.float64) * _sigmoid(gate)[..., None]


def gate_backward(g, y, gate):
    """-> (dy, dgate)."""
    g, y = np.asarray(g, np.float64), np.asarray(y, np.float64)
    s = _sigmoid(gate)
    return g * s[..., None], (g * y).sum(-1) * s * (1.0 - s)
