"""Generate ``whole_model_tiny.npz``: nanolab's own GPT on a tiny shape.

Run once, in a container where the reference checkout is importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_whole_model_golden.py /path/to/reference

Builds ``nanolab.model.GPT`` (``nanolab/model.py:205``) from ``build_config`` with the
architecture defaults (QK-norm, RoPE, gated attention, value residual, SwiGLU, tied
embeddings), overwrites every parameter with seeded N(0, 0.05) values (so the
zero-initialised projections and gates take part), runs one fp32 forward + backward
on CPU, and stores the parameters, the token ids, the loss and every gradient.  One
plain-causal case with GQA and one sliding-window case.  The test-suite reads the
file; it never imports the reference.
"""
from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).parent


def one(build_config, build_model, tag, overrides, out):
    cfg = build_config(None, dict(
        n_layer=2, d_model=32, n_head=4, n_kv_head=2, head_dim=32, block_size=40, vocab_size=61,
        dtype="fp32", compile=False, dropout=0.0, **overrides))
    torch.manual_seed(7)
    model = build_model(cfg)
    g = torch.Generator().manual_seed(11)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.05)
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or ".norm" in name or "norm_f" in name:
                p.add_(1.0)
    idx = torch.randint(0, cfg.vocab_size, (2, cfg.block_size), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, cfg.block_size), generator=g)
    model.train()
    logits, loss = model(idx, tgt)
    loss.backward()
    out[f"{tag}/idx"] = idx.numpy()
    out[f"{tag}/tgt"] = tgt.numpy()
    out[f"{tag}/loss"] = np.float64(loss.item())
    out[f"{tag}/logits"] = logits.detach().numpy()
    for name, p in model.named_parameters():
        out[f"{tag}/param/{name}"] = p.detach().numpy()
        if p.grad is not None:
            out[f"{tag}/grad/{name}"] = p.grad.numpy()
    print(tag, "loss", loss.item(), "params", sum(p.numel() for p in model.parameters()))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from nanolab.config import build_config
    from nanolab.model import build_model
    out = {}
    one(build_config, build_model, "causal", {}, out)
    one(build_config, build_model, "swa", dict(mixer="swa", swa_window=16, swa_sinks=2), out)
    np.savez_compressed(HERE / "whole_model_tiny.npz", **out)


if __name__ == "__main__":
    main(sys.argv[1])
