"""TEST INFRASTRUCTURE -- float64 restatement of the attention core of nanolab's KV-cached
block forward.  Never imported by the product path.

``Attention.forward_cached`` (``nanolab/mixers.py:372-467``) attends the active block's
queries to [cache | block] with a mask it builds from absolute positions:

* sliding window (``:417-432``): keep ``kpos <= qpos`` and
  (``kpos > qpos - (window - sinks)`` or ``kpos < sinks``); after eviction the cached keys'
  positions are no longer contiguous, which is why positions, not offsets, define the mask;
* causal block without a window (``:433-437``): everything in the cache, lower-triangular
  inside the block -- with contiguous positions that is ``kpos <= qpos``;
* neither (block diffusion): every key.

Parity pinned: ``tests/golden/cached_forward.npz`` records what nanolab's own
``forward_hidden_window`` passed to and got from SDPA over several committed blocks
(``tests/golden/make_cached_golden.py``); ``tests/test_cached_forward.py`` holds ``keep_mask``
to nanolab's masks exactly and ``forward`` to SDPA's results at 1e-12.
"""
from __future__ import annotations

import numpy as np


def keep_mask(qpos, kpos, causal: bool, window: int = 0, sinks: int = 0) -> np.ndarray:
    """``[T, L]`` boolean keep-mask from absolute positions."""
    qp = np.asarray(qpos, dtype=np.int64)[:, None]
    kp = np.asarray(kpos, dtype=np.int64)[None, :]
    if window > 0:
        return (kp <= qp) & ((kp > qp - (window - sinks)) | (kp < sinks))
    if causal:
        return kp <= qp
    return np.ones((qp.shape[0], kp.shape[1]), dtype=bool)


def forward(q, k, v, scale: float, qpos, kpos, causal: bool, window: int = 0, sinks: int = 0):
    """q ``[B,T,H,D]``, k / v ``[B,Hkv,L,D]`` (nanolab's cache layout) -> (y ``[B,T,H,D]``, lse ``[B,H,T]``)."""
    q, k, v = (np.asarray(t, dtype=np.float64) for t in (q, k, v))
    B, T, H, D = q.shape
    group = H // k.shape[1]
    keep = keep_mask(qpos, kpos, causal, window, sinks)
    y = np.zeros_like(q)
    lse = np.full((B, H, T), -np.inf)
    for b in range(B):
        for h in range(H):
            s = q[b, :, h] @ k[b, h // group].T * scale            # [T, L]
            s = np.where(keep, s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            m = np.where(np.isfinite(m), m, 0.0)
            p = np.exp(s - m)
            l = p.sum(axis=1, keepdims=True)
            ok = l[:, 0] > 0
            y[b, ok, h] = (p[ok] / l[ok]) @ v[b, h // group]
            lse[b, h, ok] = (m[ok, 0] + np.log(l[ok, 0]))
    return y, lse
