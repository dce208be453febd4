"""Generate ``qk_prologue.npz``: nanolab's own q/k prologue in float64.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_prologue_golden.py /path/to/reference

Runs nanolab's ``RMSNorm`` (``nanolab/mixers.py:46-56``), ``build_rope_cache`` (``:59-65``)
and ``apply_rope`` (``:68-75``) on seeded bf16-rounded inputs upcast to float64, and
differentiates them with autograd.  Inputs are stored as bf16 bit patterns so the same
values feed every kernel dtype exactly.  The test-suite reads the file; it never imports
the reference.
"""
from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).parent
# (B, T, H, D, norm, rope)
CASES = [(2, 37, 3, 64, True, True), (1, 50, 2, 32, True, True), (1, 19, 2, 128, True, True),
         (2, 16, 2, 64, True, False), (2, 16, 2, 64, False, True)]


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from nanolab import mixers
    out = {}
    for n, (B, T, H, D, norm, rope) in enumerate(CASES):
        g = torch.Generator().manual_seed(2000 + n)
        x = (torch.randn(B, T, H, D, generator=g) * 1.7).bfloat16()
        gy = torch.randn(B, T, H, D, generator=g).bfloat16()
        w = (1.0 + 0.3 * torch.randn(D, generator=g)).bfloat16()
        bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
        xa = x.double().requires_grad_()
        y = xa
        mod = None
        if norm:
            mod = mixers.RMSNorm(D).double()
            with torch.no_grad():
                mod.weight.copy_(w.double())
            y = mod(y)
        cos = sin = None
        if rope:
            cos, sin = mixers.build_rope_cache(T, D, 10000.0, "cpu", torch.float64)
            y = mixers.apply_rope(y, cos, sin)
        y.backward(gy.double())
        tag = f"case{n}"
        out[f"{tag}/meta"] = np.array([B, T, H, D, int(norm), int(rope)])
        out[f"{tag}/x"], out[f"{tag}/gy"], out[f"{tag}/w"] = bits(x), bits(gy), bits(w)
        out[f"{tag}/y"] = y.detach().numpy()
        out[f"{tag}/dx"] = xa.grad.numpy()
        if norm:
            out[f"{tag}/dw"] = mod.weight.grad.numpy()
        if rope:
            out[f"{tag}/cos"], out[f"{tag}/sin"] = cos.numpy(), sin.numpy()
    np.savez_compressed(HERE / "qk_prologue.npz", **out)
    print("wrote", len(CASES), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
