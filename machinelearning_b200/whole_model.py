"""The caller of the attention path: nanolab's GPT training step, restated.

nanolab's own ``model.py`` / ``train.py`` use ``flash_cuda`` unchanged, but they
are not part of this package, so the whole-model configuration (12 layers,
d_model 768, 12 heads of 64, RoPE, RMSNorm, SwiGLU, vocabulary 50304, context
1024, global batch 64 sequences) needs a caller that lives here.  This module is
that caller and nothing more: the same layer arithmetic and the same parameter
names as ``nanolab/model.py:178-245`` (``Block``, ``GPT``) and
``nanolab/mixers.py:206-345`` (``Attention``), so a nanolab ``state_dict`` loads
into it, and ``tests/golden/whole_model_tiny.npz`` (written by
``tests/golden/make_whole_model_golden.py`` from nanolab itself) pins its loss and
gradients to nanolab's.

The attention core goes through ``mixer_glue.attention_core`` -- the routing of
``Attention._flash_cuda_attn`` (``nanolab/mixers.py:347-370``) -- and falls back
to SDPA exactly where nanolab's mixer does (CPU tensors, flag off).

``DataParallelStep`` is the data-parallel training step of the whole-model
configuration: one process per GPU, each on ``global_batch / world`` sequences,
gradients averaged with one ``all_reduce`` per flat bucket (the convention of
the reference's only data-parallel script: average every gradient that exists),
then a fused AdamW step.  nanolab's phase-1 preset trains with Muon + AdamW;
the optimiser is not on the attention path and AdamW stands in for it here.
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import flash_cuda, mixer_glue, qk_prologue, value_gate


@dataclasses.dataclass
class ModelShape:
    """The fields of nanolab's ``Config`` (``nanolab/config.py:47-255``) this path reads.

    Defaults are the ``phase1`` preset (``config.py:393-399``) with nanolab's
    architecture defaults: QK-norm, gated attention, value residual, tied
    embeddings, zero-initialised output projections.
    """
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    n_kv_head: int = 0          # 0 -> n_head
    head_dim: int = 64
    vocab_size: int = 50304
    block_size: int = 1024
    rope_base: float = 10000.0
    qk_norm: bool = True
    gated_attention: bool = True
    value_residual: bool = True
    tie_embeddings: bool = True
    zero_init_proj: bool = True
    flash_cuda: bool = False    # ``--flash_cuda true`` (config.py:233-239)
    swa_window: int = 0         # > 0: every layer is the SWA mixer (config.py:127-139)
    swa_sinks: int = 0
    fused_prologue: bool = True  # with flash_cuda on: QK-norm + RoPE + cast in one kernel (qk_prologue)
    fused_epilogue: bool = True  # with flash_cuda on: value blend and head gate in one kernel each (value_gate)

    def __post_init__(self):
        if self.n_kv_head == 0:
            self.n_kv_head = self.n_head
        if self.n_head % self.n_kv_head:
            raise ValueError("n_head must be a multiple of n_kv_head")

    @property
    def ffn_hidden(self) -> int:
        """SwiGLU width: 2/3 of 4·d rounded up to 64 (``config.py:364-368``)."""
        return (int(2 / 3 * 4 * self.d_model) + 63) // 64 * 64


class RMSNorm(nn.Module):
    """``nanolab/mixers.py:46-56``: weight only, eps 1e-6."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(T: int, head_dim: int, base: float, device, dtype):
    """cos / sin ``[T, head_dim]``, both halves the same angles (``mixers.py:59-65``)."""
    half = torch.arange(0, head_dim, 2, device=device).float() / head_dim
    ang = torch.outer(torch.arange(T, device=device).float(), base ** -half)
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rotate(x, cos, sin):
    """Rotary embedding on ``[B,T,H,D]``, half-split convention (``mixers.py:68-75``)."""
    lo, hi = x.chunk(2, dim=-1)
    return x * cos[None, :, None, :] + torch.cat((-hi, lo), dim=-1) * sin[None, :, None, :]


class Attention(nn.Module):
    """Projections, QK-norm, RoPE, value residual, attention core, gate, output projection."""

    def __init__(self, s: ModelShape):
        super().__init__()
        self.H, self.Hkv, self.D = s.n_head, s.n_kv_head, s.head_dim
        self.attn_scale = 1.0 / math.sqrt(s.head_dim)
        self.q_proj = nn.Linear(s.d_model, self.H * self.D, bias=False)
        self.k_proj = nn.Linear(s.d_model, self.Hkv * self.D, bias=False)
        self.v_proj = nn.Linear(s.d_model, self.Hkv * self.D, bias=False)
        self.o_proj = nn.Linear(self.H * self.D, s.d_model, bias=False)
        if s.qk_norm:
            self.q_norm, self.k_norm = RMSNorm(self.D), RMSNorm(self.D)
        else:
            self.q_norm = self.k_norm = None
        self.gate = nn.Linear(s.d_model, self.H, bias=True) if s.gated_attention else None
        self.vr_lambda = nn.Parameter(torch.zeros(1)) if s.value_residual else None
        # what mixer_glue.decline_reason reads off a mixer
        self.flash_cuda = bool(s.flash_cuda)
        self.causal = True
        self.block_attn = 0
        self.swa_window, self.swa_sinks = int(s.swa_window), int(s.swa_sinks)
        self._flash_declined = False
        self.fused_prologue = bool(s.fused_prologue)
        self.fused_epilogue = bool(s.fused_epilogue)

    def _prologue(self, q, k, cos, sin):
        """QK-norm and RoPE (``mixers.py:287-292``): one fused kernel per tensor when this step goes
        through the kernels anyway, the separate tensor passes otherwise."""
        qw = None if self.q_norm is None else self.q_norm.weight
        kw = None if self.k_norm is None else self.k_norm.weight
        if (self.fused_prologue and self.flash_cuda and qk_prologue.supports(q, qw, cos, sin)
                and qk_prologue.supports(k, kw, cos, sin) and flash_cuda.is_available()):
            return qk_prologue.qk_prologue(q, qw, cos, sin), qk_prologue.qk_prologue(k, kw, cos, sin)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        return rotate(q, cos, sin), rotate(k, cos, sin)

    def _sdpa(self, q, k, v):
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        if self.Hkv != self.H:
            k = k.repeat_interleave(self.H // self.Hkv, dim=1)
            v = v.repeat_interleave(self.H // self.Hkv, dim=1)
        if self.swa_window:
            T = q.shape[2]
            i = torch.arange(T, device=q.device)
            span = self.swa_window - self.swa_sinks
            keep = (i[None, :] <= i[:, None]) & ((i[None, :] > i[:, None] - span) | (i[None, :] < self.swa_sinks))
            y = F.scaled_dot_product_attention(q, k, v, attn_mask=keep, scale=self.attn_scale)
        else:
            y = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=self.attn_scale)
        return y.transpose(1, 2).contiguous()

    def forward(self, x, cos, sin, v0):
        B, T, _ = x.shape
        q = self.q_proj(x).view(B, T, self.H, self.D)
        k = self.k_proj(x).view(B, T, self.Hkv, self.D)
        v = raw_v = self.v_proj(x).view(B, T, self.Hkv, self.D)
        q, k = self._prologue(q, k, cos, sin)
        fused = self.fused_epilogue and self.flash_cuda and x.is_cuda and flash_cuda.is_available()
        if self.vr_lambda is not None and v0 is not None:
            if fused and value_gate.supports_blend(v, v0, self.vr_lambda):
                v = value_gate.value_blend(v, v0, self.vr_lambda)
            else:
                lam = torch.sigmoid(self.vr_lambda)
                v = (1 - lam) * v + lam * v0
        y = mixer_glue.attention_core(self, q, k, v, self.attn_scale)
        if y is None:
            y = self._sdpa(q, k, v)
        if self.gate is not None:
            logits = self.gate(x)
            if fused and value_gate.supports_gate(y, logits):
                y = value_gate.head_gate(y, logits)
            else:
                y = y * torch.sigmoid(logits).unsqueeze(-1)
        return self.o_proj(y.reshape(B, T, self.H * self.D)), raw_v


class SwiGLU(nn.Module):
    """``down(silu(gate(x)) * up(x))`` (``nanolab/model.py:29-43``)."""

    def __init__(self, s: ModelShape):
        super().__init__()
        self.gate = nn.Linear(s.d_model, s.ffn_hidden, bias=False)
        self.up = nn.Linear(s.d_model, s.ffn_hidden, bias=False)
        self.down = nn.Linear(s.ffn_hidden, s.d_model, bias=False)

    def forward(self, x):
        return self.down(F.silu(self.gate(x)) * self.up(x))


class Block(nn.Module):
    """Pre-norm residual block (``nanolab/model.py:178-193``)."""

    def __init__(self, s: ModelShape):
        super().__init__()
        self.norm1, self.mixer = RMSNorm(s.d_model), Attention(s)
        self.norm2, self.ffn = RMSNorm(s.d_model), SwiGLU(s)

    def forward(self, x, cos, sin, v0):
        mixed, raw_v = self.mixer(self.norm1(x), cos, sin, v0)
        x = x + mixed
        return x + self.ffn(self.norm2(x)), raw_v


class GPT(nn.Module):
    """Embedding, blocks, final norm, tied head, mean cross-entropy (``model.py:205-245``, ``:364-453``)."""

    def __init__(self, s: ModelShape):
        super().__init__()
        self.shape = s
        self.tok_emb = nn.Embedding(s.vocab_size, s.d_model)
        self.blocks = nn.ModuleList(Block(s) for _ in range(s.n_layer))
        self.norm_f = RMSNorm(s.d_model)
        self.lm_head = nn.Linear(s.d_model, s.vocab_size, bias=False)
        if s.tie_embeddings:
            self.lm_head.weight = self.tok_emb.weight
        for m in self.modules():           # weights N(0, 0.02), biases 0 (model.py:245-251)
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)
        for b in self.blocks:
            if b.mixer.gate is not None:   # gate starts at 0.5 (mixers.py:247-249)
                nn.init.zeros_(b.mixer.gate.weight)
            if s.zero_init_proj:           # blocks start as the identity (model.py:263-285)
                nn.init.zeros_(b.mixer.o_proj.weight)
                nn.init.zeros_(b.ffn.down.weight)
        self._rope = {}

    def n_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self) -> float:
        """nanolab's estimate, 6·N + 12·L·H·D·T (``model.py:461-490``)."""
        s = self.shape
        span = min(s.swa_window, s.block_size) if s.swa_window else s.block_size
        return 6.0 * self.n_params() + 12.0 * s.n_layer * s.n_head * s.head_dim * span

    def forward(self, idx, targets=None):
        s = self.shape
        x = self.tok_emb(idx)
        key = (idx.shape[1], x.device, x.dtype)
        if key not in self._rope:
            self._rope[key] = rope_tables(idx.shape[1], s.head_dim, s.rope_base, x.device, x.dtype)
        cos, sin = self._rope[key]
        v0 = None
        for blk in self.blocks:
            x, raw_v = blk(x, cos, sin, v0)
            if v0 is None:
                v0 = raw_v                 # layer 0's values anchor every later layer
        x = self.norm_f(x)
        if targets is None:
            return self.lm_head(x[:, [-1], :]), None
        logits = self.lm_head(x)
        loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), ignore_index=-1)
        return logits, loss


class _Bucket:
    """A flat fp32 buffer that holds the gradients of a run of parameters (their ``.grad`` are views of it)."""

    def __init__(self, params, device):
        self.params = params
        self.flat = torch.zeros(sum(p.numel() for p in params), dtype=torch.float32, device=device)
        self.pending = len(params)
        self.launched = False
        offset = 0
        for p in params:
            p.grad = self.flat[offset:offset + p.numel()].view_as(p)
            offset += p.numel()


class DataParallelStep:
    """One optimiser step of the whole-model configuration on this rank's share of the batch.

    ``step(idx, targets)``: autocast forward, backward, gradient average across
    ranks, global-norm clip (nanolab's default 1.0, ``config.py:163``), fused AdamW.
    The average is the reference's only data-parallel convention, a per-gradient
    all-reduce (``Rust_MLKit/arch_02_value_resid/train_gpt_sprint_native.py:1407``,
    ``:1916``, ``:2006``: ``if p.grad is not None: all_reduce(p.grad, AVG)``), done in
    flat fp32 buckets of ``bucket_mb`` and overlapped with the backward: the
    parameters' gradients are views of the buckets (nothing is packed or unpacked),
    a hook on every parameter counts its bucket down, and when the last gradient of
    a bucket has arrived the bucket's ``all_reduce`` is launched on a side stream
    while autograd carries on with the earlier layers.  The main stream joins the
    side stream before the clip.  Buckets follow the order in which gradients
    appear (last layer first).  Which parameters take part is learnt from the first
    step, which averages without overlap -- layer 0's ``vr_lambda`` never gets a
    gradient (it has no ``v0``), which is why this is not a wrapper that expects
    every parameter to take part.  With one rank no collective is issued.

    ``capture(idx, targets)`` records the whole step -- forward, backward, the NCCL
    all-reduces, the clip and the optimiser -- into one CUDA graph; ``step`` then copies
    the batch into the graph's input buffers and replays it.  A step is about two
    thousand kernel launches; at 8 GPUs (8 sequences per GPU) the host cannot issue them as
    fast as the GPU finishes them, and one replay removes that bound.  The capture runs
    three warm-up steps first with the learning rate at zero and clears the optimiser
    state afterwards, so parameters and state are those of an uncaptured run.
    """

    def __init__(self, model: GPT, lr: float = 6e-4, weight_decay: float = 0.1, grad_clip: float = 1.0,
                 dtype=torch.bfloat16, bucket_mb: int = 32, group=None, overlap: bool = True):
        self.model, self.grad_clip, self.dtype, self.group = model, grad_clip, dtype, group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.bucket_elems = bucket_mb * (1 << 20) // 4
        self.overlap = overlap
        params = list(model.parameters())
        decay = [p for p in params if p.dim() >= 2]
        rest = [p for p in params if p.dim() < 2]
        on_gpu = params[0].is_cuda
        # on the GPU the learning rate is a device tensor: a captured step reads it at replay time
        self.lr = torch.tensor(float(lr), device=params[0].device) if on_gpu else float(lr)
        self.opt = torch.optim.AdamW(
            [dict(params=decay, weight_decay=weight_decay), dict(params=rest, weight_decay=0.0)],
            lr=self.lr, betas=(0.9, 0.95), fused=on_gpu, capturable=on_gpu)
        self.collectives = 0
        self._graph = None
        self._buckets = None                 # built after the first backward
        self._bucket_of = {}
        self._hooks = []
        self._comm = torch.cuda.Stream(device=params[0].device) if on_gpu and self.world > 1 else None

    # ---- gradient averaging -------------------------------------------------------------------
    def _build_buckets(self) -> None:
        """After the first backward: the parameters that received a gradient, in the order their gradients
        appear (the reverse of registration), packed into flat buffers that own the gradients from now on."""
        got = [p for p in reversed(list(self.model.parameters())) if p.grad is not None]
        first = {id(p): p.grad for p in got}
        self._buckets, run, used = [], [], 0
        for p in got:
            if run and used + p.numel() > self.bucket_elems:
                self._buckets.append(run)
                run, used = [], 0
            run.append(p)
            used += p.numel()
        if run:
            self._buckets.append(run)
        self._buckets = [_Bucket(ps, got[0].device) for ps in self._buckets]
        for b in self._buckets:
            for p in b.params:
                p.grad.copy_(first[id(p)])                        # this step's gradients move in
                self._bucket_of[id(p)] = b
                self._hooks.append(p.register_post_accumulate_grad_hook(self._grad_arrived))

    def _grad_arrived(self, p) -> None:
        b = self._bucket_of[id(p)]
        b.pending -= 1
        if b.pending == 0 and self.overlap:
            self._launch(b)

    def _launch(self, b: _Bucket) -> None:
        b.launched = True
        self.collectives += 1
        if self._comm is None:                                    # CPU ranks: nothing to overlap with
            dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group)
            b.flat.mul_(1.0 / self.world)
            return
        self._comm.wait_stream(torch.cuda.current_stream())       # the bucket's last gradient has been written
        with torch.cuda.stream(self._comm):
            dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group)
            b.flat.mul_(1.0 / self.world)

    def average_gradients(self) -> None:
        """Called after the backward: launches what the hooks have not (every bucket on the first step or
        without overlap; a bucket one of whose parameters got no gradient this time) and joins the side stream."""
        if self.world == 1:
            return
        if self._buckets is None:
            self._build_buckets()
        for b in self._buckets:
            if not b.launched:
                self._launch(b)
        if self._comm is not None:
            torch.cuda.current_stream().wait_stream(self._comm)

    def close(self) -> None:
        """Detach from the model: remove the gradient hooks (they hold this object, and through it a captured
        graph with NCCL kernels, alive past ``del``) and drop the graph and the buckets.  Call it before the
        process group is destroyed."""
        for h in self._hooks:
            h.remove()
        self._hooks, self._bucket_of, self._graph = [], {}, None
        if self._buckets is not None:
            for b in self._buckets:
                for p in b.params:
                    p.grad = None
            self._buckets = None

    def _zero_grad(self) -> None:
        if self._buckets is None:
            self.opt.zero_grad(set_to_none=True)
            return
        for b in self._buckets:                                   # the gradients stay views of the buckets
            b.flat.zero_()
            b.pending, b.launched = len(b.params), False

    def capture(self, idx, targets) -> None:
        """Record one whole step into a CUDA graph (GPU only); later ``step`` calls replay it."""
        if not idx.is_cuda:
            raise ValueError("capture needs CUDA tensors")
        self._idx, self._tgt = idx.clone(), targets.clone()
        lr = self.lr.clone()
        self.lr.zero_()                                   # warm-up steps must not move the parameters
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self._eager_step(self._idx, self._tgt)
        torch.cuda.current_stream().wait_stream(side)
        for state in self.opt.state.values():             # in place: the graph keeps these tensors
            for t in state.values():
                if torch.is_tensor(t):
                    t.zero_()
        self.lr.copy_(lr)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._loss = self._eager_step(self._idx, self._tgt)
        self._graph = graph

    def step(self, idx, targets) -> torch.Tensor:
        if self._graph is not None:
            self._idx.copy_(idx, non_blocking=True)
            self._tgt.copy_(targets, non_blocking=True)
            self._graph.replay()
            return self._loss
        return self._eager_step(idx, targets)

    def _eager_step(self, idx, targets) -> torch.Tensor:
        dev = idx.device.type
        with torch.autocast(dev, dtype=self.dtype, enabled=self.dtype != torch.float32):
            _, loss = self.model(idx, targets)
        loss.backward()
        self.average_gradients()
        torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.grad_clip)
        self.opt.step()
        self._zero_grad()
        return loss.detach()


def synthetic_tokens(vocab_size: int, batch: int, block_size: int, seed: int = 0):
    """Token ids uniform in ``[0, vocab)`` from a CPU generator, inputs = targets
    (``nanolab/bench_gpu.py:35-38``)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randint(0, vocab_size, (batch, block_size), generator=g)
    return x, x.clone()


def _flag(text: str) -> bool:
    """nanolab's CLI spells booleans ``true`` / ``false`` (``nanolab/config.py:487-505``)."""
    if text.lower() in ("true", "1", "yes"):
        return True
    if text.lower() in ("false", "0", "no"):
        return False
    raise ValueError(f"expected true or false, got {text!r}")


def main(argv=None) -> int:
    """Synthetic-token micro-benchmark of the training step, after ``nanolab/bench_gpu.py:41-110``.

        python -m machinelearning_b200.whole_model --flash_cuda true [--batch_size 16 --iters 10 --swa_window 0]

    Prints tokens/s, ms per step, the model-FLOPs estimate nanolab uses and the loss, for one GPU.
    """
    import argparse
    import json
    import time
    ap = argparse.ArgumentParser()
    ap.add_argument("--flash_cuda", type=_flag, default=False)
    ap.add_argument("--fused_prologue", type=_flag, default=True)
    ap.add_argument("--batch_size", type=int, default=16)
    ap.add_argument("--swa_window", type=int, default=0)
    ap.add_argument("--swa_sinks", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device")
    torch.manual_seed(0)
    shape = ModelShape(flash_cuda=a.flash_cuda, fused_prologue=a.fused_prologue, swa_window=a.swa_window,
                       swa_sinks=a.swa_sinks)
    model = GPT(shape).cuda()
    step = DataParallelStep(model)
    x, y = (t.cuda() for t in synthetic_tokens(shape.vocab_size, a.batch_size, shape.block_size))
    for _ in range(a.warmup):
        loss = step.step(x, y)
    torch.cuda.synchronize()
    t0 = time.time()
    for _ in range(a.iters):
        loss = step.step(x, y)
    torch.cuda.synchronize()
    sec = (time.time() - t0) / a.iters
    tokens = a.batch_size * shape.block_size
    print(json.dumps({"flash_cuda": a.flash_cuda, "fused_prologue": a.fused_prologue and a.flash_cuda,
                      "tok_s": tokens / sec, "ms_per_step": sec * 1e3, "loss": loss.item(),
                      "params_m": model.n_params() / 1e6, "flops_per_tok": model.flops_per_token(),
                      "model_tflops": model.flops_per_token() * tokens / sec / 1e12,
                      "kernel_declined": any(b.mixer._flash_declined for b in model.blocks)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
