"""B200 flash attention behind nanolab's ``flash_cuda`` module interface.

Drop-in for ``nanolab/flash_cuda.py``: same public names, same call signatures,
same exceptions.  What is different underneath:

* the native side is a C-ABI shared library (``libnlfa.so``, ``include/nlfa.h``)
  called through ctypes, not a pybind11 module built by ninja;
* Python owns every buffer (outputs, the logsumexp tape, the backward's Delta
  scratch) so torch's caching allocator and stream semantics apply;
* ``use_mma`` still picks the kernel family (reference: ``flash_cuda.py:233-279``):
  ``False`` is the fp32 SIMT kernels, ``True`` demands the tensor-core kernels
  (TMA + tcgen05 + TMEM, sm_100a), ``None`` takes them whenever dtype and head dim
  allow and the load-time self-test passed;
* ``flash_attn`` also takes keyword-only ``window`` / ``sinks`` -- the mixer's
  sliding-window mask (``nanolab/mixers.py:96-135``) runs inside the kernel with
  masked key blocks skipped, instead of declining to SDPA (``mixers.py:357``).

There is no CPU path here: when the library or a CUDA device is missing,
``is_available()`` is False with a reason and ``flash_attn`` raises.

    python -m machinelearning_b200.flash_cuda        # self-check, then timings
"""
from __future__ import annotations

import logging
import math
import os

import torch

from . import _lib

log = logging.getLogger("machinelearning_b200.flash_cuda")

SUPPORTED_HEAD_DIMS = (32, 64, 128)
SUPPORTED_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
MMA_DTYPES = (torch.float16, torch.bfloat16)      # tcgen05 kind::f16 operands
# Head dims with a tensor-core kernel, forward and backward alike (32 runs the
# 64-wide kernels on tiles that TMA pads with zeros).  The reference stops its
# tensor-core backward at 64 (flash_cuda.py:48-51).
MMA_HEAD_DIMS = (32, 64, 128)
MMA_BWD_HEAD_DIMS = (32, 64, 128)
_PROBE_HEAD_DIMS = (64, 128)                      # kernel instantiations the load-time probe runs
# Backward layout on the tensor-core path at head dims up to 64: the reference's two independent
# passes, or -- with NLFA_FUSED_BACKWARD=1 -- one pass that forms dQ inside the dK/dV pass.  Both
# are bit-reproducible; on B200 the two passes are the faster ones at these head dims (the one
# pass saves the second computation of P and dS but pays for a reduction of dQ across CTAs).
FUSED_BACKWARD = os.environ.get("NLFA_FUSED_BACKWARD", "0") == "1"

_DTYPE_CODE = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16,
               torch.bfloat16: _lib.DTYPE_BF16}

_ext = None
_load_error: str | None = None
_load_attempted = False
_mma_ok = False
_mma_error: str | None = None
_status_words: dict[int, torch.Tensor] = {}       # device index -> pinned int32 word the kernels write


def _watch_device(lib, index: int) -> None:
    """Give the library a page-locked word for device ``index`` (once per device).  A kernel whose
    bounded wait runs out writes its code there, so the next call learns of it from host memory,
    with no synchronisation on the hot path."""
    if index in _status_words:
        return
    import ctypes
    word = torch.zeros(1, dtype=torch.int32).pin_memory()
    with torch.cuda.device(index):
        st = lib.nlfa_set_status_mirror(word.data_ptr())
    _lib.check("nlfa_set_status_mirror", st)
    word.view = ctypes.c_uint.from_address(word.data_ptr())      # read without going through torch
    _status_words[index] = word


def device_timed_out() -> bool:
    """True when a kernel on any watched device has given up a wait since the last reset."""
    if torch.compiler.is_compiling():          # a traced caller is checked when it runs, by the C entry points
        return False
    return any(w.view.value != 0 for w in _status_words.values())


def reset_device_status() -> int:
    """Read and clear the status word of every watched device (synchronises them).  Returns the
    last non-zero raw word seen, 0 when there was none.  After this the kernels run again."""
    import ctypes
    seen = 0
    lib = _load()
    if lib is None:
        return 0
    for index in list(_status_words):
        raw = ctypes.c_uint(0)
        with torch.cuda.device(index):
            lib.nlfa_device_status(ctypes.byref(raw))
        seen = raw.value or seen
    return seen


def _probe_mma(lib) -> tuple[bool, str]:
    """Run the tensor-core self-test on the device (reference: ``_probe_mma``,
    ``flash_cuda.py:59-88``).  Fails closed: the tensor-core path stays off."""
    try:
        if not lib.nlfa_device_supported():
            major, minor = torch.cuda.get_device_capability()
            return False, f"tcgen05 needs sm_100, this device is sm_{major}{minor}"
        import ctypes
        ws = torch.empty(lib.nlfa_selftest_workspace_bytes(), dtype=torch.uint8, device="cuda")
        errs = (ctypes.c_float * 2)()
        stream = torch.cuda.current_stream().cuda_stream
        for code, name in ((_lib.DTYPE_BF16, "bf16"), (_lib.DTYPE_F16, "f16")):
            for d in _PROBE_HEAD_DIMS:
                st = lib.nlfa_selftest(code, d, ws.data_ptr(), ws.numel(), errs, stream)
                if st != _lib.OK:
                    return False, (f"self-test failed for {name} D={d}: {_lib.strerror(st)} "
                                   f"(S err {errs[0]:.3e}, O err {errs[1]:.3e})")
        return True, ""
    except Exception as e:                                    # noqa: BLE001
        return False, f"{type(e).__name__}: {e}"


def _load():
    """Load the library once.  Never raises (reference: ``flash_cuda.py:91-135``);
    callers gate on ``is_available()``."""
    global _ext, _load_error, _load_attempted, _mma_ok, _mma_error
    if _load_attempted:
        return _ext
    _load_attempted = True
    if os.environ.get("NANOLAB_FLASH_CUDA", "1") == "0":
        _load_error = "disabled by NANOLAB_FLASH_CUDA=0"
        return None
    if not torch.cuda.is_available():
        _load_error = "no CUDA device"
        return None
    try:
        _ext = _lib.load()
    except Exception as e:                                    # noqa: BLE001
        _ext = None
        _load_error = f"{type(e).__name__}: {e}"
        log.warning("libnlfa did not load (%s)", _load_error)
        return None
    _mma_ok, _mma_error = _probe_mma(_ext)
    if not _mma_ok:
        log.warning("tensor-core path off (%s); using the SIMT kernels", _mma_error)
    try:
        _watch_device(_ext, torch.cuda.current_device())
    except Exception as e:                                    # noqa: BLE001
        log.warning("status word not mirrored to the host (%s)", e)
    return _ext


_TIMED_OUT = ("a kernel gave up a bounded wait (status 10: a bounded wait inside a kernel gave up); "
              "outputs of that launch are not valid; call reset_device_status() to re-arm")


def is_available() -> bool:
    """True once the library is loaded on a machine with a CUDA device -- and no kernel has given
    up a wait since the last ``reset_device_status()``: like the reference's loader
    (``flash_cuda.py:91-135``) this fails closed, so the mixer falls back instead of training on."""
    return _load() is not None and not device_timed_out()


def unavailable_reason() -> str:
    _load()
    if _ext is None:
        return _load_error or "unknown"
    return _TIMED_OUT if device_timed_out() else ""


def mma_available() -> bool:
    """True when the tensor-core kernels are usable: library loaded and the
    on-device self-test passed."""
    return _load() is not None and _mma_ok


def mma_unavailable_reason() -> str:
    if _load() is None:
        return unavailable_reason()
    return "" if _mma_ok else (_mma_error or "unknown")


def effective_dtype(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.dtype | None:
    """The dtype the kernel would run at (reference: ``flash_cuda.py:161-177``):
    the autocast dtype under an enabled CUDA autocast, else the common dtype."""
    if q.is_cuda and torch.is_autocast_enabled("cuda"):
        return torch.get_autocast_dtype("cuda")
    if q.dtype == k.dtype == v.dtype:
        return q.dtype
    return None


def supports(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """Shape / dtype / device gate (reference: ``flash_cuda.py:180-202``).  Does
    not load the library."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        return False
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        return False
    if effective_dtype(q, k, v) not in SUPPORTED_DTYPES:
        return False
    if q.shape[-1] not in SUPPORTED_HEAD_DIMS:
        return False
    if k.shape[:2] != q.shape[:2] or v.shape[:2] != q.shape[:2]:
        return False
    if k.shape[2] != v.shape[2] or k.shape[3] != q.shape[3] or v.shape[3] != q.shape[3]:
        return False
    if k.shape[2] == 0 or q.shape[2] % k.shape[2] != 0:
        return False
    return True


def check_window(window: int, sinks: int, block: int = 0) -> None:
    """Same refusals as ``sliding_window_mask`` (``nanolab/mixers.py:119-123``), and the mixer's for a
    block-causal mask next to a window (``mixers.py:300-304``)."""
    if block < 0:
        raise ValueError(f"block length must be >= 0, got {block}")
    if block and window:
        raise ValueError("block-causal (diffusion) attention and SWA are mutually exclusive masks")
    if window == 0:
        if sinks:
            raise ValueError("swa sinks set without a window")
        return
    if window < 1:
        raise ValueError(f"swa window must be >=1, got {window}")
    if not 0 <= sinks < window:
        raise ValueError(f"swa sinks must satisfy 0 <= sinks < window, "
                         f"got sinks={sinks} window={window}")


class _on_device:
    """``torch.cuda.device(index)`` when ``index`` is not the current device, else nothing: the
    context manager costs several microseconds per call, the comparison a fraction of one."""
    __slots__ = ("guard",)

    def __init__(self, index: int):
        self.guard = None if index == torch.cuda.current_device() else torch.cuda.device(index)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _stream_of(index: int) -> int:
    """The raw handle of torch's current stream on device ``index``."""
    return torch._C._cuda_getCurrentRawStream(index)


def fwd(q, k, v, scale: float, use_mma: bool, window: int = 0, sinks: int = 0, block: int = 0):
    """(O, LSE) through the C ABI.  Contiguous same-dtype CUDA tensors only
    (reference native entry: ``flash_attn_cuda.cu:1655-1704``).  ``block > 0``: the block-causal mask
    of ``nanolab/mixers.py:78-93`` instead of the causal one."""
    lib = _load()
    if lib is None:
        raise RuntimeError(f"flash_cuda is unavailable ({unavailable_reason()})")
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    index = q.device.index
    if index not in _status_words:
        _watch_device(lib, index)
    o = torch.empty_like(q)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    with _on_device(index):
        st = lib.nlfa_fwd_masked(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                 B, T, H, Hkv, D, float(scale), int(window), int(sinks), int(block),
                                 _DTYPE_CODE[q.dtype],
                                 _lib.PATH_TENSOR if use_mma else _lib.PATH_SIMT,
                                 _stream_of(index))
    if st:
        _lib.check("nlfa_fwd", st)
    return o, lse


def bwd(dout, q, k, v, o, lse, scale: float, use_mma: bool, window: int = 0, sinks: int = 0,
        fused: bool | None = None, block: int = 0):
    """(dQ, dK, dV) through the C ABI (reference: ``flash_attn_cuda.cu:1744-1813``).

    ``fused`` picks the backward's layout on the tensor-core path at head dims up to 64: the
    reference's two independent passes (``nlfa_bwd``; the default) or one pass that forms dQ inside
    the dK/dV pass (``nlfa_bwd_fused``).  Both are bit-reproducible.  Elsewhere there are only the
    two passes."""
    lib = _load()
    if lib is None:
        raise RuntimeError(f"flash_cuda is unavailable ({unavailable_reason()})")
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    index = q.device.index
    if index not in _status_words:
        _watch_device(lib, index)
    can_fuse = bool(use_mma) and D <= 64
    if fused is None:
        fused = can_fuse and FUSED_BACKWARD
    elif fused and not can_fuse:
        raise ValueError("the fused backward exists on the tensor-core path for head dims up to 64")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    nbytes = lib.nlfa_bwd_fused_scratch_bytes(B, T, H, D) if fused else lib.nlfa_bwd_scratch_bytes(B, T, H)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    passes = (_lib.PASS_DELTA | _lib.PASS_FUSED) if fused else _lib.PASS_ALL
    with _on_device(index):
        st = lib.nlfa_bwd_masked(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                 lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                 scratch.data_ptr(), scratch.numel(), B, T, H, Hkv, D, float(scale),
                                 int(window), int(sinks), int(block), _DTYPE_CODE[q.dtype],
                                 _lib.PATH_TENSOR if use_mma else _lib.PATH_SIMT, passes,
                                 _stream_of(index))
    if st:
        _lib.check("nlfa_bwd_masked", st)
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    """Causal / windowed GQA attention on [B,T,H,D] with the taped LSE carried to
    backward (reference: ``flash_cuda.py:205-230``)."""

    @staticmethod
    def forward(ctx, q, k, v, scale, use_mma, window, sinks, block=0):
        o, lse = fwd(q, k, v, scale, use_mma, window, sinks, block)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = float(scale)
        ctx.use_mma = bool(use_mma)
        ctx.window, ctx.sinks, ctx.block = int(window), int(sinks), int(block)
        return o

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = bwd(dout.contiguous(), q, k, v, o, lse, ctx.scale, ctx.use_mma,
                         ctx.window, ctx.sinks, block=ctx.block)
        return dq, dk, dv, None, None, None, None, None


def _tensor_path_fits(dtype, head_dim) -> bool:
    return dtype in MMA_DTYPES and head_dim in MMA_HEAD_DIMS


def prepare(q, k, v, scale, use_mma, window, sinks, block=0):
    """The checks, defaults and casts of ``flash_attn`` (reference: ``flash_cuda.py:251-278``);
    returns ``(q, k, v, scale, use_mma)`` ready for the kernels."""
    if not supports(q, k, v):
        raise ValueError(
            "flash_cuda.flash_attn: unsupported inputs "
            f"(q={tuple(q.shape)}/{q.dtype}, k={tuple(k.shape)}/{k.dtype}, "
            f"v={tuple(v.shape)}/{v.dtype}); head_dim must be one of "
            f"{SUPPORTED_HEAD_DIMS} and the effective dtype one of "
            f"{SUPPORTED_DTYPES}")
    check_window(window, sinks, block)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    dtype = effective_dtype(q, k, v)
    q = q.to(dtype).contiguous()
    k = k.to(dtype).contiguous()
    v = v.to(dtype).contiguous()

    fits = _tensor_path_fits(dtype, q.shape[-1])
    if use_mma is None:
        use_mma = fits and mma_available()
    elif use_mma:
        if dtype not in MMA_DTYPES:
            raise ValueError(
                f"flash_cuda: use_mma=True but the effective dtype is {dtype}; "
                f"the tensor-core kernels exist only for {MMA_DTYPES}")
        if q.shape[-1] not in MMA_HEAD_DIMS:
            raise ValueError(
                f"flash_cuda: use_mma=True but head_dim is {q.shape[-1]}; "
                f"the tensor-core kernels exist only for {MMA_HEAD_DIMS}")
        if not mma_available():
            raise RuntimeError(
                f"flash_cuda: use_mma=True but the tensor-core path is "
                f"unavailable ({mma_unavailable_reason()})")
    return q, k, v, scale, use_mma


def flash_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
               scale: float | None = None, use_mma: bool | None = None, *,
               window: int = 0, sinks: int = 0, block: int = 0) -> torch.Tensor:
    """Causal GQA flash attention. q [B,T,H,D], k/v [B,T,Hkv,D] -> [B,T,H,D].

    Same contract as the reference (``flash_cuda.py:233-279``): raises
    ``ValueError`` for unsupported inputs instead of falling back; casts q/k/v to
    the effective dtype and makes them contiguous as autograd ops.  ``window`` /
    ``sinks`` select the sliding-window mask; ``window=0`` is plain causal.  ``block > 0``
    selects the block-causal mask of nanolab's diffusion / semi-autoregressive mode instead
    (``nanolab/mixers.py:78-93``: a query sees its own block of ``block`` positions and every
    earlier one; ``block >= T`` is fully bidirectional attention); it excludes a window.
    """
    q, k, v, scale, use_mma = prepare(q, k, v, scale, use_mma, window, sinks, block)
    if torch.compiler.is_compiling():
        from . import compile_ops              # registered operators: one graph node instead of a graph break
        return compile_ops.attn_fwd(q, k, v, float(scale), bool(use_mma), int(window), int(sinks), int(block))[0]
    if not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)):
        return fwd(q, k, v, scale, use_mma, window, sinks, block)[0]       # inference: no autograd node
    return _FlashAttnFn.apply(q, k, v, scale, use_mma, window, sinks, block)


def flash_attn_cached(q: torch.Tensor, k_full: torch.Tensor, v_full: torch.Tensor, scale: float | None = None, *,
                      qpos: torch.Tensor | None = None, kpos: torch.Tensor | None = None, causal: bool = False,
                      window: int = 0, sinks: int = 0, return_lse: bool = False, use_mma: bool | None = None):
    """Attention of an active block over [cache | block]: the core of nanolab's ``forward_cached``.

    ``q [B,T,H,D]`` is the active block; ``k_full`` / ``v_full [B,Hkv,L,D]`` are the cache with the
    block's own keys appended, in nanolab's cache layout (``nanolab/mixers.py:401-405``), narrow KV
    heads; ``qpos [T]`` / ``kpos [L]`` are absolute positions (``None``: contiguous, the block last).
    The mask is the one ``forward_cached`` builds (``mixers.py:417-437``): with a window, the
    sliding-window mask on positions (``causal`` must be set, as nanolab requires); with
    ``causal``, full to the cache and lower-triangular in the block; otherwise every key.
    Forward only (nanolab runs this path under ``no_grad``); returns ``[B,T,H,D]`` (and the
    logsumexp ``[B,H,T]`` with ``return_lse``).  Raises ``ValueError`` for unsupported inputs.
    ``use_mma`` as in ``flash_attn``: ``None`` lets the library take its tensor-core kernel where it
    applies (16-bit inputs, a block of at least 16 rows per KV head over at least 256 keys) and the fp32
    kernel elsewhere; ``False`` / ``True`` force one (``True`` raises where it does not apply).
    """
    ok = (q.dim() == 4 and k_full.dim() == 4 and v_full.dim() == 4 and q.is_cuda and k_full.is_cuda and v_full.is_cuda
          and q.dtype == k_full.dtype == v_full.dtype and q.dtype in SUPPORTED_DTYPES
          and q.shape[-1] in SUPPORTED_HEAD_DIMS and k_full.shape == v_full.shape
          and k_full.shape[0] == q.shape[0] and k_full.shape[3] == q.shape[3]
          and k_full.shape[1] > 0 and q.shape[2] % k_full.shape[1] == 0)
    if not ok:
        raise ValueError(f"flash_attn_cached: unsupported inputs (q={tuple(q.shape)}/{q.dtype}, "
                         f"k={tuple(k_full.shape)}/{k_full.dtype}, v={tuple(v_full.shape)}/{v_full.dtype})")
    check_window(window, sinks)
    if window and not causal:
        raise ValueError("cached SWA decode requires causal=True")          # nanolab/mixers.py:410-414
    B, T, H, D = q.shape
    Hkv, L = k_full.shape[1], k_full.shape[2]
    if qpos is None and T > L:
        raise ValueError("without positions the block must be the last T of the L keys")
    lib = _load()
    if lib is None:
        raise RuntimeError(f"flash_cuda is unavailable ({unavailable_reason()})")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    pos = lambda t, n: None if t is None else t.detach().to(device=q.device, dtype=torch.int32).reshape(n).contiguous()
    qp, kp = pos(qpos, T), pos(kpos, L)
    q, k_full, v_full = q.detach().contiguous(), k_full.detach().contiguous(), v_full.detach().contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device) if return_lse else None
    nbytes = lib.nlfa_fwd_cached_scratch_bytes(B, T, H, Hkv, L, D)      # > 0: the keys are split over CTAs
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device) if nbytes else None
    with _on_device(q.device.index):
        path = _lib.PATH_AUTO if use_mma is None else (_lib.PATH_TENSOR if use_mma else _lib.PATH_SIMT)
        st = lib.nlfa_fwd_cached_path(q.data_ptr(), k_full.data_ptr(), v_full.data_ptr(), o.data_ptr(),
                                      None if lse is None else lse.data_ptr(),
                                      None if qp is None else qp.data_ptr(), None if kp is None else kp.data_ptr(),
                                      B, T, H, Hkv, L, D, float(scale), int(bool(causal)), int(window), int(sinks),
                                      _DTYPE_CODE[q.dtype], path, None if scratch is None else scratch.data_ptr(),
                                      nbytes, _stream_of(q.device.index))
    if st == 7 and use_mma:
        raise ValueError("flash_attn_cached: use_mma=True but the tensor-core kernel does not apply to these inputs")
    _lib.check("nlfa_fwd_cached", st)
    return (o, lse) if return_lse else o


def sdpa_reference(q, k, v, scale):
    """nanolab's attention without the kernel (the role of the reference's ``sdpa_reference``,
    ``flash_cuda.py:282-294``): torch SDPA on ``[B,H,T,D]`` views with the KV heads repeated for
    the group.  The self-check's comparison arm; ``flash_attn`` never calls it."""
    heads_per_kv = q.shape[2] // k.shape[2]
    widen = (lambda t: t) if heads_per_kv == 1 else (lambda t: t.repeat_interleave(heads_per_kv, dim=2))
    out = torch.nn.functional.scaled_dot_product_attention(
        q.permute(0, 2, 1, 3), widen(k).permute(0, 2, 1, 3), widen(v).permute(0, 2, 1, 3),
        is_causal=True, scale=scale)
    return out.permute(0, 2, 1, 3).contiguous()


def _median_ms(fn, iters: int, warmup: int = 5) -> float:
    """Median device time of ``fn`` in milliseconds: one CUDA-event pair per call, each call
    synchronised, after ``warmup`` untimed calls (what the reference's ``_bench_once`` reports)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for first, last in pairs:
        first.record()
        fn()
        last.record()
        last.synchronize()
    ms = sorted(first.elapsed_time(last) for first, last in pairs)
    mid = len(ms) // 2
    return ms[mid] if len(ms) % 2 else 0.5 * (ms[mid - 1] + ms[mid])


def _cached_check(args) -> int:
    """``--cached BLOCK``: the KV-cached block forward against what ``forward_cached`` does today
    (``nanolab/mixers.py:401-460``: ``torch.cat`` of cache and block, ``repeat_interleave``, a boolean mask,
    SDPA), causal block, same GPU."""
    import torch.nn.functional as F
    dtype = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[args.dtype]
    B, L, H, Hkv, D, T = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim, args.cached
    w, s = args.window, args.sinks
    torch.manual_seed(0)
    q = torch.randn(B, T, H, D, device="cuda", dtype=dtype)
    k = torch.randn(B, Hkv, L, D, device="cuda", dtype=dtype)
    v = torch.randn_like(k)
    ck, cv, kt, vt = (t.contiguous() for t in (k[:, :, :L - T], v[:, :, :L - T], k[:, :, L - T:], v[:, :, L - T:]))
    apos, kpos = torch.arange(L - T, L, device="cuda"), torch.arange(L, device="cuda")
    scale = 1.0 / math.sqrt(D)

    def nanolab_way():
        kf, vf = torch.cat([ck, kt], 2), torch.cat([cv, vt], 2)
        if w:
            keep = (kpos[None, :] <= apos[:, None]) & ((kpos[None, :] > apos[:, None] - (w - s)) | (kpos[None, :] < s))
        else:
            keep = torch.cat([torch.ones(T, L - T, dtype=torch.bool, device="cuda"),
                              torch.tril(torch.ones(T, T, dtype=torch.bool, device="cuda"))], 1)
        rep = H // Hkv
        if rep > 1:
            kf, vf = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
        y = F.scaled_dot_product_attention(q.transpose(1, 2), kf, vf, attn_mask=keep[None, None], scale=scale)
        return y.transpose(1, 2).contiguous()

    def kernel_with_cat():
        return flash_attn_cached(q, torch.cat([ck, kt], 2), torch.cat([cv, vt], 2), scale, causal=True,
                                 window=w, sinks=s)

    def kernel_only():
        return flash_attn_cached(q, k, v, scale, causal=True, window=w, sinks=s)

    err = (kernel_only().float() - nanolab_way().float()).abs().max().item()
    print(f"block {T} over {L} keys, B{B} H{H}/{Hkv} D{D} {args.dtype} window {w} sinks {s}: max |diff| {err:.3e}")
    kv_bytes = 2 * k.numel() * k.element_size()
    for name, fn in (("cat + repeat + mask + SDPA", nanolab_way), ("cat + flash_attn_cached", kernel_with_cat),
                     ("flash_attn_cached", kernel_only)):
        ms = _median_ms(fn, args.iters)
        print(f"  {name:28s} {ms * 1e3:9.1f} us   {kv_bytes / ms / 1e6:8.0f} GB/s of K, V")
    return 0


_CLI_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def _cli_args():
    import argparse
    ap = argparse.ArgumentParser(description="self-check against torch SDPA, then timings")
    for flag, default in (("--batch", 8), ("--seq", 1024), ("--heads", 12), ("--kv_heads", 4),
                          ("--head_dim", 32), ("--iters", 20), ("--window", 0), ("--sinks", 0)):
        ap.add_argument(flag, type=int, default=default)
    ap.add_argument("--dtype", default="bf16", choices=tuple(_CLI_DTYPES))
    ap.add_argument("--cached", type=int, default=0, metavar="BLOCK",
                    help="instead: a BLOCK-token active block over --seq keys through flash_attn_cached, "
                         "against nanolab's cat + repeat_interleave + masked SDPA")
    return ap.parse_args()


def main() -> int:
    """``python -m machinelearning_b200.flash_cuda``: the job of the reference's self-check
    (``flash_cuda.py:315-379``, same flags and default shape B8 T1024 H12/4 D32 bf16): agreement
    with SDPA is printed before any timing, then forward and forward+backward medians per arm."""
    args = _cli_args()
    if not torch.cuda.is_available():
        print("no CUDA device -- nothing to run")
        return 1
    if not is_available():
        print(f"library unavailable: {unavailable_reason()}")
        return 1
    if args.cached:
        return _cached_check(args)

    dtype = _CLI_DTYPES[args.dtype]
    shape_q = (args.batch, args.seq, args.heads, args.head_dim)
    shape_kv = (args.batch, args.seq, args.kv_heads, args.head_dim)
    torch.manual_seed(0)
    q, k, v = (torch.randn(sh, device="cuda", dtype=dtype, requires_grad=True)
               for sh in (shape_q, shape_kv, shape_kv))
    upstream = torch.randn(shape_q, device="cuda", dtype=dtype)
    scale = 1.0 / math.sqrt(args.head_dim)
    tensor_cores = mma_available() and _tensor_path_fits(dtype, args.head_dim)
    print(f"q {shape_q} k/v {shape_kv} {args.dtype}; tensor-core kernels "
          + ("on" if tensor_cores else f"off ({mma_unavailable_reason() or 'dtype / head dim'})"))

    arms = {"SDPA": lambda: sdpa_reference(q, k, v, scale),
            "simt": lambda: flash_attn(q, k, v, scale, use_mma=False)}
    if tensor_cores:
        arms["tc"] = lambda: flash_attn(q, k, v, scale, use_mma=True)

    def with_grads(arm):
        out = arm()
        return out, torch.autograd.grad(out, (q, k, v), upstream)

    want, want_grads = with_grads(arms["SDPA"])
    for name, arm in arms.items():
        if name == "SDPA":
            continue
        got, got_grads = with_grads(arm)
        worst_grad = max(float((g.float() - w.float()).abs().max()) for g, w in zip(got_grads, want_grads))
        print(f"{name:>5} - SDPA   max|O| {float((got.float() - want.float()).abs().max()):.3e}   "
              f"max|grad| {worst_grad:.3e}")

    rows = [(name, _median_ms(arm, args.iters), _median_ms(lambda arm=arm: with_grads(arm), args.iters))
            for name, arm in arms.items()]
    sdpa_fwd, sdpa_both = rows[0][1], rows[0][2]
    print(f"{'':>5} {'forward':>11} {'fwd + bwd':>11} {'speed-up over SDPA':>22}")
    for name, t_fwd, t_both in rows:
        print(f"{name:>5} {t_fwd:9.3f}ms {t_both:9.3f}ms {sdpa_fwd / t_fwd:10.2f}x {sdpa_both / t_both:9.2f}x")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
