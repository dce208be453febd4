"""The CPU oracle against the reference-generated golden vectors (CPU only)."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_f64 as orc
from oracle import sdpa_port


def test_oracle_matches_reference_golden(golden):
    g = golden
    o, lse = orc.attention_fwd(g["q"], g["k"], g["v"], g["scale"], g["window"], g["sinks"], g["block"])
    dq, dk, dv = orc.attention_bwd(g["dout"], g["q"], g["k"], g["v"], g["scale"],
                                   g["window"], g["sinks"], g["block"])
    # same bar the reference holds its own CPU mirror to (nanolab/tests.py:280-293)
    for name, got in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert np.abs(got - g[name]).max() < 1e-12, f"{g['name']}: {name}"


def test_delta_is_rowsum_of_do_times_o(golden):
    g = golden
    delta = orc.attention_delta(g["o"], g["dout"])
    want = (g["dout"].astype(np.float64) * g["o"]).sum(-1).transpose(0, 2, 1)
    assert np.abs(delta - want).max() < 1e-12


def test_mask_position_by_position():
    # nanolab/tests.py:2992-3017 walks the mask the same way
    T, w, s = 40, 8, 2
    keep = orc.keep_mask(T, w, s)
    for q in range(T):
        for k in range(T):
            want = k <= q and (k > q - (w - s) or k < s)
            assert keep[q, k] == want, (q, k)
    assert keep.sum(axis=1).max() <= w


def test_window_at_least_T_is_plain_causal():
    # nanolab/tests.py:3020-3051
    T = 50
    assert (orc.keep_mask(T, T, 0) == orc.keep_mask(T)).all()
    assert (orc.keep_mask(T, 4 * T, 3) == orc.keep_mask(T)).all()
    assert not (orc.keep_mask(T, 8, 0) == orc.keep_mask(T)).all()


@pytest.mark.parametrize("w,s", [(0, 1), (4, 4), (4, 5), (-1, 0)])
def test_invalid_window_refused(w, s):
    # nanolab/tests.py:3083-3118
    with pytest.raises(ValueError):
        orc.keep_mask(16, w, s)


def test_pairs_and_flops():
    assert orc.unmasked_pairs(1024) == 1024 * 1025 // 2
    assert orc.unmasked_pairs(4096, 256, 0) == 1015936
    for T, w, s in ((300, 64, 4), (65, 64, 4), (128, 32, 1), (100, 400, 4)):
        assert orc.unmasked_pairs(T, w, s) == int(orc.keep_mask(T, w, s).sum())
    f, b = orc.attention_flops(32, 1024, 12, 64)
    assert abs((f + b) / 1e9 - 180.56) < 0.01


@pytest.mark.parametrize("window,sinks", [(0, 0), (64, 4), (32, 0), (400, 4)])
def test_cpu_baseline_port_agrees_with_oracle(window, sinks):
    # the timed CPU path (torch SDPA, chunked SWA) computes the same function
    torch.manual_seed(0)
    B, T, H, Hkv, D = 1, 300, 4, 2, 32
    q, k, v, do = (torch.randn(B, T, h, D, dtype=torch.float64)
                   for h in (H, Hkv, Hkv, H))
    scale = 1.0 / math.sqrt(D)
    y, dq, dk, dv = sdpa_port.cpu_fwd_bwd(q, k, v, do, scale, window, sinks)
    o, _ = orc.attention_fwd(q, k, v, scale, window, sinks)
    gq, gk, gv = orc.attention_bwd(do, q, k, v, scale, window, sinks)
    for got, want in ((y, o), (dq, gq), (dk, gk), (dv, gv)):
        assert np.abs(got.numpy() - want).max() < 1e-10


def test_chunk_choice_mirrors_reference_rule():
    # nanolab/mixers.py:160-165
    assert sdpa_port.auto_chunk(4096, 256) == 256
    assert sdpa_port.auto_chunk(2048, 64) == 256
    assert sdpa_port.auto_chunk(512, 256) == 0
    assert sdpa_port.auto_chunk(2048, 512) == 512
