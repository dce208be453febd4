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
    and hands every other step to nanolab's own ``forward`` untouched; ``forward_cached`` (the KV-cached
    block forward of the samplers, ``mixers.py:372-467``) likewise goes through ``flash_attn_cached``.  At nanolab's 124M shape the
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


_PLAIN_FORWARD: dict[type, tuple] = {}        # mixer class -> the (forward, forward_cached) it had before fuse_mixer()


def fused_attention_forward(self, x, cos, sin, v0=None):
    """``Attention.forward`` of nanolab (``mixers.py:280-345``) for a step the kernels take: the same
    projections, then one kernel each for QK-norm + RoPE + cast, the value-residual blend
    (``mixers.py:294-297``) and the head gate (``mixers.py:340-342``) around the attention core.  Same
    return value ``(o_proj(y), raw_v)``.  A step the kernels decline -- flag off, CPU tensors, shapes or
    masks they do not take, library not loaded or timed out -- goes to the class's own ``forward``,
    with nanolab's own warnings and errors."""
    from . import qk_prologue, value_gate
    plain = _PLAIN_FORWARD[next(c for c in type(self).__mro__ if c in _PLAIN_FORWARD)][0]
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


# Query rows x keys below which a cached block forward stays with nanolab's own lines (0: every block
# goes through the kernels).  Even a single sequence in 32-token blocks gains -- nanolab's own
# `sample_blockwise_cached` on the 124M model: 683 -> 746 tokens/s, `forward_hidden_window` alone 1.6x --
# because such blocks are bound by the host's launches and the fused path makes a third as many; the knob
# is for callers whose host path differs.
CACHED_MIN_WORK = 0


def _cached_step_declined(self, x, causal, cache) -> bool:
    """The cached block forward stays with nanolab's own lines when the flag is off, off the GPU, while
    gradients are recorded (the kernel is forward only; nanolab's samplers run under ``no_grad``), for a
    window without ``causal`` (nanolab raises for it, ``mixers.py:410-414``), for dtypes / head dims
    the kernels do not take, and for blocks too small to be worth it (``CACHED_MIN_WORK``)."""
    if not (getattr(self, "flash_cuda", False) and x.is_cuda) or torch.is_grad_enabled():
        return True
    if self.swa_window and not causal:
        return True
    held = cache.get("k")
    keys = x.shape[1] + (0 if held is None else held.shape[2])
    if x.shape[0] * x.shape[1] * self.n_head * keys < CACHED_MIN_WORK:
        return True
    dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
    if dtype not in flash_cuda.SUPPORTED_DTYPES or self.head_dim not in flash_cuda.SUPPORTED_HEAD_DIMS:
        return True
    return not flash_cuda.is_available()


def fused_attention_forward_cached(self, x, cos, sin, v0, cache, commit, causal=False):
    """``Attention.forward_cached`` of nanolab (``mixers.py:372-467``) with the kernels: the active
    block's projections, QK-norm + RoPE and value blend as in ``fused_attention_forward``, then
    ``flash_attn_cached`` over [cache | block] -- the mask comes from absolute positions, so neither the
    boolean mask nor the ``repeat_interleave`` of the KV heads is built -- and the head gate.  The cache
    keeps nanolab's layout and bookkeeping (``k`` / ``v [B,Hkv,L,D]``; with a window ``pos`` and ``end``,
    and on commit only the sinks and the tail the next block can still reach are kept), so nanolab's
    samplers see no difference."""
    from . import qk_prologue, value_gate
    cls = next(c for c in type(self).__mro__ if c in _PLAIN_FORWARD)
    if _cached_step_declined(self, x, causal, cache):
        return _PLAIN_FORWARD[cls][1](self, x, cos, sin, v0, cache, commit, causal)
    B, T, _ = x.shape
    H, Hkv, D = self.n_head, self.n_kv_head, self.head_dim
    q = self.q_proj(x).view(B, T, H, D)
    k = self.k_proj(x).view(B, T, Hkv, D)
    v = raw_v = self.v_proj(x).view(B, T, Hkv, D)
    qw = self.q_norm.weight if self.qk_norm else None
    kw = self.k_norm.weight if self.qk_norm else None
    if ((qw is not None or cos is not None) and qk_prologue.supports(q, qw, cos, sin)
            and qk_prologue.supports(k, kw, cos, sin)):
        q = qk_prologue.qk_prologue(q, qw, cos, sin, self.q_norm.eps if self.qk_norm else qk_prologue.EPS)
        k = qk_prologue.qk_prologue(k, kw, cos, sin, self.k_norm.eps if self.qk_norm else qk_prologue.EPS)
    else:
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        if cos is not None:
            rope = sys.modules[cls.__module__].apply_rope
            q, k = rope(q, cos, sin), rope(k, cos, sin)
    if self.value_residual and v0 is not None:
        if value_gate.supports_blend(v, v0, self.vr_lambda):
            v = value_gate.value_blend(v, v0, self.vr_lambda)
        else:
            lam = torch.sigmoid(self.vr_lambda)
            v = (1 - lam) * v + lam * v0
    if not (q.dtype == k.dtype == v.dtype):                  # (an autocast region that cast only some of them)
        k, v = k.to(q.dtype), v.to(q.dtype)

    # [cache | block] in the cache's layout
    block_k, block_v = k.transpose(1, 2), v.transpose(1, 2)                     # [B,Hkv,T,D]
    old_k, old_v = cache.get("k"), cache.get("v")
    k_full = block_k.contiguous() if old_k is None else torch.cat([old_k.to(q.dtype), block_k], dim=2)
    v_full = block_v.contiguous() if old_v is None else torch.cat([old_v.to(q.dtype), block_v], dim=2)

    window, sinks = int(self.swa_window or 0), int(self.swa_sinks or 0)
    qpos = kpos = None
    if window:
        # absolute positions: after an eviction the cache is shorter than the prefix it stands for
        first = int(cache.get("end", 0))
        held = cache.get("pos")
        if held is None:
            held = torch.arange(first, device=x.device)
        qpos = torch.arange(first, first + T, device=x.device)
        kpos = torch.cat([held, qpos])
    if commit:
        if window:
            last = first + T
            reach = window - sinks - 1                       # how far back the next block's first query sees
            keep = (kpos < sinks) | (kpos >= last - reach)
            cache["k"], cache["v"] = k_full[:, :, keep].detach(), v_full[:, :, keep].detach()
            cache["pos"], cache["end"] = kpos[keep], last
        else:
            cache["k"], cache["v"] = k_full.detach(), v_full.detach()

    y = flash_cuda.flash_attn_cached(q, k_full, v_full, self.attn_scale, qpos=qpos, kpos=kpos,
                                     causal=bool(causal), window=window, sinks=sinks)          # [B,T,H,D]
    if self.gated:
        logits = self.gate(x)
        if value_gate.supports_gate(y, logits):
            y = value_gate.head_gate(y, logits)
        else:
            y = y * torch.sigmoid(logits).unsqueeze(-1)
    return self.o_proj(y.reshape(B, T, H * D)), raw_v


def fuse_mixer(package: str = "nanolab") -> None:
    """Route ``<package>.mixers.Attention.forward`` and ``.forward_cached`` through
    ``fused_attention_forward`` / ``fused_attention_forward_cached``.  Call after ``install()``; imports
    ``<package>.mixers`` if it is not imported yet.  ``unfuse_mixer`` undoes it."""
    mixers = importlib.import_module(f"{package}.mixers")
    if getattr(mixers, "flash_cuda", None) is not flash_cuda:
        raise RuntimeError(f"{package}.mixers is bound to another flash_cuda; call install() before importing it")
    cls = mixers.Attention
    if cls.forward is fused_attention_forward:
        return
    _PLAIN_FORWARD[cls] = (cls.forward, cls.forward_cached)
    cls.forward = fused_attention_forward
    cls.forward_cached = fused_attention_forward_cached


def unfuse_mixer(package: str = "nanolab") -> None:
    mixers = sys.modules.get(f"{package}.mixers")
    cls = getattr(mixers, "Attention", None)
    if cls is not None and cls in _PLAIN_FORWARD:
        cls.forward, cls.forward_cached = _PLAIN_FORWARD.pop(cls)


def main() -> int:
    """``python -m machinelearning_b200.mixer_glue [--batch B --block T --context L]`` with nanolab
    importable: nanolab's own ``GPT.forward_hidden_window`` (phase-1 preset, bf16 autocast, random
    weights) decoding ``B`` sequences block by block with commits, on nanolab's lines and through
    ``fuse_mixer()``; wall clock, tokens/s."""
    import argparse
    import time
    ap = argparse.ArgumentParser(description="nanolab's cached block decode with and without fuse_mixer()")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--block", type=int, default=32)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--min-work", type=int, default=None,
                    help="override CACHED_MIN_WORK (0: every block through the kernels)")
    args = ap.parse_args()
    if args.min_work is not None:
        global CACHED_MIN_WORK
        CACHED_MIN_WORK = args.min_work
    if not torch.cuda.is_available() or not flash_cuda.is_available():
        print(f"nothing to run: {flash_cuda.unavailable_reason() or 'no CUDA device'}")
        return 1
    install()
    try:
        from nanolab.config import build_config
        from nanolab.model import build_model
    except ImportError as e:
        print(f"nanolab is not importable ({e}); put its parent directory on PYTHONPATH")
        return 1
    torch.manual_seed(0)
    cfg = build_config("phase1", dict(run_name="decode", block_size=max(2048, args.context), flash_cuda=True,
                                      compile=False, dtype="bf16", dropout=0.0))
    model = build_model(cfg).cuda().eval()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    tokens = torch.randint(0, 50000, (args.batch, args.context), device="cuda")

    def decode():
        caches = [{} for _ in model.blocks]
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            for start in range(0, args.context, args.block):
                model.forward_hidden_window(tokens[:, start:start + args.block], start, caches, True, True)

    def seconds():
        decode()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.reps):
            decode()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / args.reps

    unfuse_mixer()
    plain = seconds()
    fuse_mixer()
    fused = seconds()
    unfuse_mixer()
    n = args.batch * args.context
    print(f"B={args.batch} block={args.block} context={args.context}: nanolab's lines {plain * 1e3:.1f} ms "
          f"({n / plain:.0f} tokens/s), fused mixer {fused * 1e3:.1f} ms ({n / fused:.0f} tokens/s), {plain / fused:.2f}x")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
