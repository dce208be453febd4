"""Generate ``cached_forward.npz``: what nanolab's KV-cached block forward feeds to, and gets from, SDPA.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_cached_golden.py /path/to/reference

Drives nanolab's own ``GPT.forward_hidden_window`` (``nanolab/model.py:328-362``) block by block --
i.e. ``Attention.forward_cached`` (``nanolab/mixers.py:372-467``) in every layer, with commits, and for
the sliding-window arm with the cache eviction that makes key positions non-contiguous -- in float64 on a
tiny seeded model, and records every call the mixer makes to ``F.scaled_dot_product_attention``: the
query block, the pre-widening K / V (cache + block), the boolean mask nanolab built, and SDPA's result.
From the cache's own ``pos`` / ``end`` entries it also records the absolute positions of queries and keys,
which is what the kernel's entry point takes instead of a mask.  Three arms: full attention to the cache with
a bidirectional block (block diffusion), the same with a causal block (self-speculation verify), and
SWA(12, 2) with a causal block.  The test-suite reads the file; it never imports the reference.
"""
from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = pathlib.Path(__file__).parent


def run_arm(build_config, build_model, tag, overrides, causal, out, blocks=(5, 7, 4, 6)):
    cfg = build_config(None, dict(n_layer=2, d_model=32, n_head=4, n_kv_head=2, head_dim=32, block_size=64,
                                  vocab_size=61, dtype="fp32", compile=False, dropout=0.0, **overrides))
    torch.manual_seed(3)
    model = build_model(cfg).double().eval()
    g = torch.Generator().manual_seed(17)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float64) * 0.3)
    tokens = torch.randint(0, cfg.vocab_size, (2, sum(blocks)), generator=g)
    caches = [{} for _ in model.blocks]
    calls = []
    real = F.scaled_dot_product_attention

    def spy(q, k, v, attn_mask=None, is_causal=False, scale=None, **kw):
        y = real(q, k, v, attn_mask=attn_mask, is_causal=is_causal, scale=scale, **kw)
        calls.append((q, k, v, attn_mask, scale, y))
        return y

    F.scaled_dot_product_attention = spy
    try:
        start, n = 0, 0
        for blk in blocks:
            # positions of the cached keys as the FIRST layer sees them before this block is committed
            before = [(c.get("pos"), int(c.get("end", 0)), None if c.get("k") is None else c["k"].shape[2])
                      for c in caches]
            first = len(calls)
            model.forward_hidden_window(tokens[:, start:start + blk], start, caches, True, causal)
            for layer, (q, k, v, mask, scale, y) in enumerate(calls[first:]):
                cpos, end, clen = before[layer]
                if cpos is None:
                    cpos = torch.arange(clen or 0)
                qpos = torch.arange(start, start + blk)
                kpos = torch.cat([cpos, qpos])
                rep = q.shape[1] // model.cfg.n_kv_head
                name = f"{tag}/call{n}"
                out[f"{name}/q"] = q.transpose(1, 2).contiguous().numpy()                  # [B,T,H,D]
                out[f"{name}/k"] = k[:, ::rep].contiguous().numpy()                        # [B,Hkv,L,D]
                out[f"{name}/v"] = v[:, ::rep].contiguous().numpy()
                out[f"{name}/y"] = y.transpose(1, 2).contiguous().numpy()                  # [B,T,H,D]
                out[f"{name}/qpos"], out[f"{name}/kpos"] = qpos.numpy(), kpos.numpy()
                out[f"{name}/mask"] = (np.ones((blk, k.shape[2]), bool) if mask is None
                                       else mask[0, 0].numpy())
                out[f"{name}/meta"] = np.array([int(causal), overrides.get("swa_window", 0),
                                                overrides.get("swa_sinks", 0)])
                out[f"{name}/scale"] = np.float64(scale)
                n += 1
            start += blk
    finally:
        F.scaled_dot_product_attention = real
    print(tag, n, "calls; last key count", calls[-1][1].shape[2])


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from nanolab.config import build_config
    from nanolab.model import build_model
    out = {}
    run_arm(build_config, build_model, "full_bidir", {}, False, out)
    run_arm(build_config, build_model, "full_causal", {}, True, out)
    run_arm(build_config, build_model, "swa_causal", dict(mixer="swa", swa_window=12, swa_sinks=2), True, out)
    np.savez_compressed(HERE / "cached_forward.npz", **out)


if __name__ == "__main__":
    main(sys.argv[1])
