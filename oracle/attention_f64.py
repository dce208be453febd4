"""float64 brute-force attention, forward and backward, in numpy.

TEST INFRASTRUCTURE.  A restatement of the reference's brute-force oracle:

* forward  -- ``nanolab/csrc/flash_attn_sim.py:193-212`` (``reference_attention``):
  widen the KV heads, materialise the full [T,T] score matrix, mask, logsumexp,
  softmax @ V.  Returns ``(O [B,T,H,D], LSE [B,H,T])`` with a natural-log LSE.
* mask     -- ``nanolab/mixers.py:125-132`` (``sliding_window_mask``): keep
  ``k <= q`` and (``k > q - (window - sinks)`` or ``k < sinks``).  ``window == 0``
  means plain causal (the reference's ``Attention`` without ``swa_window``);
  ``window >= T`` degenerates to plain causal (``mixers.py:117-118``).
* block-causal mask -- ``nanolab/mixers.py:78-93`` (``block_causal_mask``): with
  ``blk = position // block``, keep ``blk[q] >= blk[k]`` (bidirectional inside a
  block, causal across blocks); it excludes a window (``mixers.py:300-304``).
* backward -- the reference differentiates its forward with autograd
  (``nanolab/tests.py:386-388``).  Here the same gradients are written out in
  closed form, the algebra of ``flash_attn_cuda.cu:1265-1482``:
  ``Delta = rowsum(dO * O)``, ``dV = P^T dO``, ``dP = dO V^T``,
  ``dS = P * (dP - Delta) * scale``, ``dQ = dS K``, ``dK = dS^T Q``, with the
  GQA group summed into the shared KV head.

Everything is float64; inputs of any float dtype are upcast first, which is how
the reference feeds bf16-rounded inputs to its oracle (``tests.py:386``).
"""
from __future__ import annotations

import numpy as np


def keep_mask(T: int, window: int = 0, sinks: int = 0, block: int = 0) -> np.ndarray:
    """[T,T] boolean keep-mask, rows = queries, columns = keys.

    Mirrors ``sliding_window_mask`` (``nanolab/mixers.py:119-132``) including its
    argument checks; ``window == 0`` is the plain causal mask, or, with ``block > 0``,
    ``block_causal_mask`` (``mixers.py:88-91``).
    """
    i = np.arange(T)
    q, k = i[:, None], i[None, :]
    causal = k <= q
    if block:
        if window:
            raise ValueError("block-causal (diffusion) attention and SWA are mutually exclusive masks")
        blk = i // block
        return blk[:, None] >= blk[None, :]
    if window == 0:
        if sinks:
            raise ValueError("swa sinks set without a window")
        return causal
    if window < 1:
        raise ValueError(f"swa window must be >=1, got {window}")
    if not 0 <= sinks < window:
        raise ValueError(f"swa sinks must satisfy 0 <= sinks < window, "
                         f"got sinks={sinks} window={window}")
    keep = causal & (k > q - (window - sinks))
    if sinks:
        keep = keep | (causal & (k < sinks))
    return keep


def unmasked_pairs(T: int, window: int = 0, sinks: int = 0, block: int = 0) -> int:
    """Number of (query, key) pairs one head attends to: the FLOP count's unit."""
    if block:
        return int(keep_mask(T, block=block).sum())
    if window == 0:
        return T * (T + 1) // 2
    span = window - sinks
    qpos = np.arange(T)
    recent_lo = np.maximum(0, qpos - span + 1)
    # recent keys, plus the sinks that are not already inside the window
    return int(((qpos - recent_lo + 1) + np.minimum(sinks, recent_lo)).sum())


def attention_flops(B: int, T: int, H: int, D: int, window: int = 0,
                    sinks: int = 0) -> tuple[float, float]:
    """(forward, backward) algorithmic FLOPs: 2 and 5 GEMMs over the unmasked pairs."""
    pairs = unmasked_pairs(T, window, sinks)
    return 4.0 * D * pairs * B * H, 10.0 * D * pairs * B * H


def _f64(x) -> np.ndarray:
    if hasattr(x, "detach"):                 # a torch tensor
        x = x.detach().to("cpu").double().numpy()
    return np.asarray(x, dtype=np.float64)


def attention_fwd(q, k, v, scale: float, window: int = 0, sinks: int = 0, block: int = 0):
    """(O [B,T,H,D], LSE [B,H,T]) in float64.  q [B,T,H,D], k/v [B,T,Hkv,D]."""
    q, k, v = _f64(q), _f64(k), _f64(v)
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    group = H // Hkv
    keep = keep_mask(T, window, sinks, block)
    o = np.empty((B, T, H, D))
    lse = np.empty((B, H, T))
    for b in range(B):
        for h in range(H):
            hk = h // group
            s = (q[b, :, h] @ k[b, :, hk].T) * scale
            s = np.where(keep, s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            e = np.exp(s - m)
            l = e.sum(axis=1, keepdims=True)
            lse[b, h] = (m + np.log(l))[:, 0]
            o[b, :, h] = (e / l) @ v[b, :, hk]
    return o, lse


def attention_delta(o, dout) -> np.ndarray:
    """Delta [B,H,T] = rowsum(dO * O) (``flash_attn_cuda.cu:1234-1262``)."""
    return np.einsum("bthd,bthd->bht", _f64(o), _f64(dout))


def attention_bwd(dout, q, k, v, scale: float, window: int = 0, sinks: int = 0, block: int = 0):
    """(dQ, dK, dV) in float64, recomputing P from the inputs."""
    dout, q, k, v = _f64(dout), _f64(q), _f64(k), _f64(v)
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    group = H // Hkv
    keep = keep_mask(T, window, sinks, block)
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    for b in range(B):
        for h in range(H):
            hk = h // group
            s = (q[b, :, h] @ k[b, :, hk].T) * scale
            s = np.where(keep, s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            e = np.exp(s - m)
            p = e / e.sum(axis=1, keepdims=True)
            o = p @ v[b, :, hk]
            do = dout[b, :, h]
            delta = (do * o).sum(axis=1, keepdims=True)
            dp = do @ v[b, :, hk].T
            ds = p * (dp - delta) * scale
            dq[b, :, h] = ds @ k[b, :, hk]
            dk[b, :, hk] += ds.T @ q[b, :, h]
            dv[b, :, hk] += p.T @ do
    return dq, dk, dv


def attention_head(q, k, v, dout, b: int, h: int, scale: float,
                   window: int = 0, sinks: int = 0):
    """One (b, h) slice of a large problem: O, LSE, dQ and this head's dK/dV share.

    For full-size workloads where the whole float64 problem is too slow: the
    caller samples heads.  With GQA the returned dK/dV are only head ``h``'s
    contribution to its KV head.
    """
    sl = lambda x, hh: _f64(x[b:b + 1, :, hh:hh + 1])
    group = q.shape[2] // k.shape[2]
    qq, kk, vv, dd = sl(q, h), sl(k, h // group), sl(v, h // group), sl(dout, h)
    o, lse = attention_fwd(qq, kk, vv, scale, window, sinks)
    dq, dk, dv = attention_bwd(dd, qq, kk, vv, scale, window, sinks)
    return o[0, :, 0], lse[0, 0], dq[0, :, 0], dk[0, :, 0], dv[0, :, 0]
