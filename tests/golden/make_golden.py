"""Generate the golden vectors that pin ``oracle/`` to the reference.

Run once, in a container where the reference checkout is importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It imports the reference's own float64 brute force
(``nanolab.csrc.flash_attn_sim.reference_attention``), differentiates it with
autograd exactly as ``nanolab/tests.py:386-388`` does, and -- for the
sliding-window cases, where the reference has no float64 function with an LSE --
applies the reference's ``sliding_window_mask`` to the same score matrix and
cross-checks the result against the reference's ``swa_chunked``.  Inputs are
rounded to bfloat16 before use and stored as their 16-bit patterns (so the same
values feed fp32, fp16-free and bf16 kernels exactly); outputs are float64.  The test-suite never imports the
reference; it reads the ``.npz`` files written here.
"""
from __future__ import annotations

import math
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).parent

# (name, B, T, H, Hkv, D, window, sinks); shapes are the ones the reference's own
# tests use (nanolab/tests.py:266-268, :313-317, :3508-3515) plus a slice of the
# fp32 correctness config.
CASES = [
    ("causal_b2_t100_h4_kv2_d32", 2, 100, 4, 2, 32, 0, 0),
    ("causal_b1_t37_h2_kv2_d32", 1, 37, 2, 2, 32, 0, 0),
    ("causal_b1_t64_h4_kv1_d32", 1, 64, 4, 1, 32, 0, 0),
    ("causal_b1_t33_h2_kv1_d32", 1, 33, 2, 1, 32, 0, 0),
    ("causal_b1_t64_h4_kv1_d64", 1, 64, 4, 1, 64, 0, 0),
    ("causal_b1_t80_h2_kv1_d128", 1, 80, 2, 1, 128, 0, 0),
    ("causal_b1_t200_h2_kv2_d64", 1, 200, 2, 2, 64, 0, 0),
    ("swa_t300_w64_s4", 1, 300, 2, 1, 32, 64, 4),
    ("swa_t300_w64_s0", 1, 300, 2, 1, 32, 64, 0),
    ("swa_t300_w256_s0", 1, 300, 1, 1, 64, 256, 0),
    ("swa_t300_w400_s4", 1, 300, 2, 1, 32, 400, 4),
    ("swa_t65_w64_s4", 1, 65, 2, 2, 32, 64, 4),
    ("swa_t128_w32_s1", 1, 128, 2, 2, 32, 32, 1),
]
# block-causal masks (nanolab/mixers.py:78-93): (name, B, T, H, Hkv, D, block); the block lengths
# straddle the kernels' 128-row tiles on purpose
BLOCK_CASES = [
    ("blockcausal_t300_b32", 1, 300, 2, 1, 64, 32),
    ("blockcausal_t300_b100", 1, 300, 2, 2, 32, 100),
    ("blockcausal_t260_b128", 1, 260, 2, 1, 64, 128),
    ("blockcausal_t200_b512", 1, 200, 2, 2, 64, 512),      # one block: fully bidirectional
    ("blockcausal_t150_b1", 1, 150, 2, 1, 32, 1),           # blocks of one: plain causal
]


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from nanolab.csrc.flash_attn_sim import reference_attention
    from nanolab import mixers

    cases = [(*c, 0) for c in CASES] + [(*c[:6], 0, 0, c[6]) for c in BLOCK_CASES]
    for seed, (name, B, T, H, Hkv, D, window, sinks, block) in enumerate(cases):
        g = torch.Generator().manual_seed(1000 + seed)
        bf = lambda *shape: torch.randn(*shape, generator=g).bfloat16()
        q, k, v, do = bf(B, T, H, D), bf(B, T, Hkv, D), bf(B, T, Hkv, D), bf(B, T, H, D)
        bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
        scale = 1.0 / math.sqrt(D)
        qa, ka, va = (t.double().requires_grad_() for t in (q, k, v))
        if window == 0 and block == 0:
            o, lse = reference_attention(qa, ka, va, scale)
        elif block:
            # reference_attention's own lines with the reference's block-causal keep-mask
            group = H // Hkv
            qs = qa.permute(0, 2, 1, 3)
            ks = ka.repeat_interleave(group, dim=2).permute(0, 2, 1, 3)
            vs = va.repeat_interleave(group, dim=2).permute(0, 2, 1, 3)
            scores = (qs @ ks.transpose(-1, -2)) * scale
            keep = mixers.block_causal_mask(T, block, "cpu", {})
            scores = scores.masked_fill(~keep, -math.inf)
            lse = torch.logsumexp(scores, dim=-1).contiguous()
            o = (torch.softmax(scores, dim=-1) @ vs).permute(0, 2, 1, 3).contiguous()
            if block == 1:                                     # must be the plain causal reference
                o_c, lse_c = reference_attention(qa.detach(), ka.detach(), va.detach(), scale)
                assert (o_c - o.detach()).abs().max() < 1e-12 and (lse_c - lse.detach()).abs().max() < 1e-12
        else:
            # reference_attention's own lines with the reference's SWA keep-mask
            group = H // Hkv
            qs = qa.permute(0, 2, 1, 3)
            ks = ka.repeat_interleave(group, dim=2).permute(0, 2, 1, 3)
            vs = va.repeat_interleave(group, dim=2).permute(0, 2, 1, 3)
            scores = (qs @ ks.transpose(-1, -2)) * scale
            keep = mixers.sliding_window_mask(T, window, sinks, "cpu", {})
            scores = scores.masked_fill(~keep, -math.inf)
            lse = torch.logsumexp(scores, dim=-1).contiguous()
            o = (torch.softmax(scores, dim=-1) @ vs).permute(0, 2, 1, 3).contiguous()
            # the reference's production SWA path must agree with this
            chunk = mixers.swa_auto_chunk(T, window) or 64
            y = mixers.swa_chunked(qs.detach(), ks.detach(), vs.detach(), window,
                                   sinks, scale, chunk).permute(0, 2, 1, 3)
            assert (y - o.detach()).abs().max() < 1e-12, name
        o.backward(do.double())
        np.savez_compressed(HERE / f"{name}.npz",
                 q=bits(q), k=bits(k), v=bits(v), dout=bits(do),
                 o=o.detach().numpy(), lse=lse.detach().numpy(),
                 dq=qa.grad.numpy(), dk=ka.grad.numpy(), dv=va.grad.numpy(),
                 meta=np.array([B, T, H, Hkv, D, window, sinks] + ([block] if block else [])),
                 scale=np.array(scale))
        print(f"wrote {name}.npz")


if __name__ == "__main__":
    main(sys.argv[1])
