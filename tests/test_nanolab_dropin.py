"""nanolab's own ``Attention`` / ``GPT`` with this package injected as ``nanolab.flash_cuda``.

The reference's caller is staged (git-ignored, built by ``oracle/build_ref.stage_nanolab``) under
``oracle/_ref/nanolab`` and imported unmodified after ``mixer_glue.install()``; nothing here is a
restatement.  Each case runs in a fresh interpreter, because ``nanolab.mixers`` binds its
``flash_cuda`` module at import time (``nanolab/mixers.py:38``).

CPU: the module identity, and the reference's own inertness test (``nanolab/tests.py:498-511``):
with the flag on and CPU tensors the mixer must decline (``mixers.py:358-370``) and give a loss
bit-identical to the flag-off model.  GPU: nanolab's ``GPT`` trained for three optimiser steps with
the flag on and off, losses compared, and every gradient compared at identical weights; then the
SWA mixer with ``_flash_cuda_attn`` routed to ``mixer_glue.attention_core``.
"""
import pathlib
import subprocess
import sys
import textwrap

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
STAGED = ROOT / "oracle" / "_ref" / "nanolab" / "mixers.py"

needs_nanolab = pytest.mark.skipif(not STAGED.exists(), reason="the reference's nanolab package is not staged "
                                                               "(python oracle/build_ref.py)")

PRELUDE = f"""
import sys, logging
sys.path.insert(0, {str(ROOT)!r})
import torch
from oracle import build_ref
assert build_ref.nanolab_on_path()
from machinelearning_b200 import mixer_glue, flash_cuda as ours
mixer_glue.install()
import nanolab.mixers as mixers
from nanolab.config import build_config
from nanolab.model import build_model
assert mixers.flash_cuda is ours, "nanolab.mixers did not bind the injected module"
import importlib
assert importlib.import_module("nanolab.flash_cuda") is ours
"""


def run_script(body: str, timeout=600):
    r = subprocess.run([sys.executable, "-c", PRELUDE + textwrap.dedent(body)], capture_output=True, text=True,
                       timeout=timeout)
    assert r.returncode == 0, f"stdout:\n{r.stdout[-3000:]}\nstderr:\n{r.stderr[-3000:]}"
    return r.stdout


@needs_nanolab
def test_flag_is_inert_on_cpu_with_the_real_mixer():
    out = run_script("""
        warnings = []
        class Grab(logging.Handler):
            def emit(self, record): warnings.append(record.getMessage())
        logging.getLogger("nanolab.mixers").addHandler(Grab())

        def toy(flag):
            torch.manual_seed(0)
            cfg = build_config(None, dict(vocab_size=256, device="cpu", dtype="fp32", n_layer=2, d_model=64, n_head=4,
                                          head_dim=16, block_size=32, batch_size=4, compile=False, mixer="attention",
                                          flash_cuda=flag))
            return build_model(cfg), cfg
        m_off, cfg = toy(False)
        m_on, _ = toy(True)
        g = torch.Generator().manual_seed(0)
        x = torch.randint(0, cfg.vocab_size, (cfg.batch_size, cfg.block_size), generator=g)
        _, loss_off = m_off(x, x.clone())
        _, loss_on = m_on(x, x.clone())
        assert torch.equal(loss_off, loss_on), "flash_cuda=True changed the CPU result"
        loss_on.backward()
        assert torch.isfinite(loss_on)
        attn = [m for m in m_on.modules() if isinstance(m, mixers.Attention)]
        assert len(attn) == 2 and all(m.flash_cuda and m._flash_declined for m in attn)
        assert len(warnings) == 2 and all("-> SDPA" in w and "unsupported inputs" in w for w in warnings), warnings
        print("inert ok")
    """)
    assert "inert ok" in out


GPU_COMMON = """
    assert ours.is_available(), ours.unavailable_reason()
    calls = {"fwd": 0, "bwd": 0}
    real_fwd, real_bwd = ours.fwd, ours.bwd
    def fwd(*a, **k):
        calls["fwd"] += 1
        return real_fwd(*a, **k)
    def bwd(*a, **k):
        calls["bwd"] += 1
        return real_bwd(*a, **k)
    ours.fwd, ours.bwd = fwd, bwd
    from nanolab.optim import build_optimizers

    def make(flag, **kw):
        torch.manual_seed(0)
        base = dict(vocab_size=512, device="cuda", dtype="bf16", n_layer=2, d_model=256, n_head=4, n_kv_head=2,
                    head_dim=64, block_size=256, batch_size=4, compile=False, mixer="attention", flash_cuda=flag,
                    grad_accum=1)
        base.update(kw)
        cfg = build_config(None, base)
        model = build_model(cfg).cuda()
        return model, cfg, build_optimizers(model, cfg)

    def one_step(model, cfg, opts, x):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = model(x, x)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), cfg.grad_clip)
        for o in opts:
            o.step()
            o.zero_grad(set_to_none=True)
        return float(loss)

    def grads_at(model, x):
        for p in model.parameters():
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = model(x, x)
        loss.backward()
        return float(loss), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}

    def compare(kw, steps=3):
        on, cfg, opt_on = make(True, **kw)
        off, _, opt_off = make(False, **kw)
        g = torch.Generator().manual_seed(1)
        x = torch.randint(0, cfg.vocab_size, (cfg.batch_size, cfg.block_size), generator=g).cuda()
        before = dict(calls)
        l_on = [one_step(on, cfg, opt_on, x) for _ in range(steps)]
        layers = cfg.n_layer
        assert calls["fwd"] - before["fwd"] == steps * layers, (calls, before)
        assert calls["bwd"] - before["bwd"] == steps * layers, (calls, before)
        l_off = [one_step(off, cfg, opt_off, x) for _ in range(steps)]
        assert calls["fwd"] - before["fwd"] == steps * layers, "the flag-off model reached the kernel"
        # losses of the two runs, step by step (the first step cannot tell: o_proj starts at zero)
        for a, b in zip(l_on, l_off):
            assert abs(a - b) <= 2e-2 * abs(b), (l_on, l_off)
        assert l_on[-1] < l_on[0], l_on
        # gradients at identical, trained (non-zero o_proj) weights
        off.load_state_dict(on.state_dict())
        loss_a, ga = grads_at(on, x)
        loss_b, gb = grads_at(off, x)
        assert abs(loss_a - loss_b) <= 2e-2 * abs(loss_b)
        assert set(ga) == set(gb) and len(ga) > 10
        worst = 0.0
        for name in ga:
            ref = gb[name].abs().max().item()
            err = (ga[name] - gb[name]).abs().max().item()
            assert err <= 2e-2 * max(ref, 1e-6), (name, err, ref)
            worst = max(worst, err / max(ref, 1e-6))
        return l_on, l_off, worst
"""


@needs_nanolab
@pytest.mark.gpu
def test_real_gpt_trains_the_same_with_the_flag_on_and_off():
    out = run_script(GPU_COMMON + """
    l_on, l_off, worst = compare({})
    print("causal ok", l_on, l_off, worst)
    """)
    assert "causal ok" in out


@needs_nanolab
@pytest.mark.gpu
def test_real_swa_mixer_through_attention_core():
    out = run_script(GPU_COMMON + """
    # the maintainer-side routing: windows go to the kernel instead of being declined (mixers.py:357)
    mixers.Attention._flash_cuda_attn = lambda self, q, k, v, scale: mixer_glue.attention_core(self, q, k, v, scale)
    l_on, l_off, worst = compare(dict(mixer="swa", swa_window=64, swa_sinks=4))
    print("swa ok", l_on, l_off, worst)
    """)
    assert "swa ok" in out


@needs_nanolab
@pytest.mark.gpu
def test_real_gpt_in_its_diffusion_modes_through_attention_core():
    """nanolab's own ``GPT.set_block_attention`` / ``set_causal(False)`` (``nanolab/model.py:295-314``):
    the block-causal and the bidirectional step go through the kernels (routing as in the SWA case) and
    give the logits of the SDPA branch."""
    out = run_script(GPU_COMMON + """
    mixers.Attention._flash_cuda_attn = lambda self, q, k, v, scale: mixer_glue.attention_core(self, q, k, v, scale)
    on, cfg, opt_on = make(True)
    off, _, _ = make(False)
    g = torch.Generator().manual_seed(2)
    x = torch.randint(0, cfg.vocab_size, (cfg.batch_size, cfg.block_size), generator=g).cuda()
    for _ in range(2):                       # off the zero-initialised output projections
        one_step(on, cfg, opt_on, x)
    off.load_state_dict(on.state_dict())
    for mode in ("block 48", "block 256 (one block)", "bidirectional"):
        for m in (on, off):
            m.set_causal(mode != "bidirectional")
            m.set_block_attention(48 if mode == "block 48" else 256 if mode.startswith("block 256") else 0)
        before = calls["fwd"]
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            la, _ = on(x, x)
            lb, _ = off(x, x)
        assert calls["fwd"] - before == cfg.n_layer, (mode, calls)
        err = (la.float() - lb.float()).abs().max().item() / lb.float().abs().max().item()
        assert err <= 2e-2, (mode, err)
        print(mode, "ok", err)
    print("diffusion ok")
    """)
    assert "diffusion ok" in out


@needs_nanolab
def test_fused_mixer_is_inert_on_cpu():
    """``mixer_glue.fuse_mixer()`` replaces nanolab's ``Attention.forward``; a step the kernels cannot take
    (CPU tensors here) must go to nanolab's own forward: loss and every gradient bit-identical to the
    unpatched class, flag on or off."""
    out = run_script("""
        def toy(flag):
            torch.manual_seed(0)
            cfg = build_config(None, dict(vocab_size=256, device="cpu", dtype="fp32", n_layer=2, d_model=64, n_head=4,
                                          n_kv_head=2, head_dim=16, block_size=32, batch_size=4, compile=False,
                                          mixer="attention", flash_cuda=flag))
            return build_model(cfg), cfg
        def run(flag):
            m, cfg = toy(flag)
            g = torch.Generator().manual_seed(0)
            x = torch.randint(0, cfg.vocab_size, (cfg.batch_size, cfg.block_size), generator=g)
            _, loss = m(x, x.clone())
            loss.backward()
            return loss.detach(), [p.grad.clone() for p in m.parameters() if p.grad is not None]
        plain = {flag: run(flag) for flag in (False, True)}
        mixer_glue.fuse_mixer()
        assert mixers.Attention.forward is mixer_glue.fused_attention_forward
        for flag in (False, True):
            loss, grads = run(flag)
            assert torch.equal(loss, plain[flag][0])
            assert len(grads) == len(plain[flag][1]) and all(torch.equal(a, b) for a, b in zip(grads, plain[flag][1]))
        mixer_glue.unfuse_mixer()
        assert mixers.Attention.forward is not mixer_glue.fused_attention_forward
        print("fused inert ok")
    """)
    assert "fused inert ok" in out


@needs_nanolab
@pytest.mark.gpu
def test_real_gpt_with_the_fused_mixer_trains_like_the_plain_one():
    """nanolab's own ``GPT`` with ``fuse_mixer()``: QK-norm + RoPE, the value-residual blend, the attention
    core and the head gate all through the kernels -- losses over three optimiser steps and every
    gradient at trained weights against the flag-off model (torch passes + SDPA), causal and SWA."""
    out = run_script(GPU_COMMON + """
    from machinelearning_b200 import qk_prologue, value_gate
    mixer_glue.fuse_mixer()
    seen = {"prologue": 0, "blend": 0, "gate": 0}
    def counting(mod, name, key):
        real = getattr(mod, name)
        def f(*a, **k):
            seen[key] += 1
            return real(*a, **k)
        setattr(mod, name, f)
    counting(qk_prologue, "qk_prologue", "prologue")
    counting(value_gate, "value_blend", "blend")
    counting(value_gate, "head_gate", "gate")
    for kw in ({}, dict(mixer="swa", swa_window=64, swa_sinks=4)):
        before = dict(seen)
        l_on, l_off, worst = compare(kw)
        # three training steps and one gradient evaluation of the flag-on model, two layers each
        assert seen["prologue"] - before["prologue"] == 4 * 2 * 2, seen       # q and k
        assert seen["gate"] - before["gate"] == 4 * 2, seen
        assert seen["blend"] - before["blend"] == 4 * 1, seen                 # the first layer has no v0
        print("fused", kw, l_on, l_off, worst)
    print("fused mixer ok")
    """)
    assert "fused mixer ok" in out


@needs_nanolab
@pytest.mark.gpu
def test_real_cached_block_forward_through_the_fused_mixer():
    """nanolab's own ``GPT.forward_hidden_window`` (``nanolab/model.py:329-362``: ``Attention.forward_cached`` in
    every layer, with commits) block by block, with and without ``fuse_mixer()``: same hidden states and the
    same caches (layout, positions, eviction), for a bidirectional block, a causal block and SWA with
    eviction, in fp32 and bf16; late blocks are long enough for the tensor-core kernel."""
    out = run_script("""
    assert ours.is_available(), ours.unavailable_reason()
    calls = {"n": 0}
    real = ours.flash_attn_cached
    def counted(*a, **k):
        calls["n"] += 1
        return real(*a, **k)
    ours.flash_attn_cached = counted
    blocks = (96, 64, 128, 32, 48)
    for dtype, tol in ((torch.float32, 2e-4), (torch.bfloat16, 3e-2)):
        for tag, kw, causal in (("bidirectional", {}, False), ("causal", {}, True),
                                ("swa", dict(mixer="swa", swa_window=64, swa_sinks=4), True)):
            torch.manual_seed(0)
            cfg = build_config(None, dict(vocab_size=512, device="cuda", dtype="fp32", n_layer=2, d_model=256,
                                          n_head=4, n_kv_head=2, head_dim=64, block_size=512, batch_size=2,
                                          compile=False, flash_cuda=True, dropout=0.0, **({"mixer": "attention"} | kw)))
            model = build_model(cfg).cuda().to(dtype).eval()
            with torch.no_grad():
                for p in model.parameters():           # off the zero-initialised projections
                    p.add_(torch.randn_like(p) * 0.02)
            g = torch.Generator().manual_seed(5)
            tokens = torch.randint(0, cfg.vocab_size, (2, sum(blocks)), generator=g).cuda()

            def drive():
                caches = [{} for _ in model.blocks]
                hidden, start = [], 0
                with torch.no_grad():
                    for n in blocks:
                        hidden.append(model.forward_hidden_window(tokens[:, start:start + n], start, caches, True, causal))
                        start += n
                return hidden, caches

            want_h, want_c = drive()
            mixer_glue.fuse_mixer()
            before = calls["n"]
            got_h, got_c = drive()
            mixer_glue.unfuse_mixer()
            assert calls["n"] - before == len(blocks) * cfg.n_layer, calls
            for a, b in zip(got_h, want_h):
                err = (a.float() - b.float()).abs().max().item() / b.float().abs().max().item()
                assert err <= tol, (tag, dtype, err)
            for ca, cb in zip(got_c, want_c):
                assert set(ca) == set(cb), (tag, set(ca), set(cb))
                assert ca["k"].shape == cb["k"].shape and ca["v"].shape == cb["v"].shape
                if "pos" in cb:
                    assert torch.equal(ca["pos"], cb["pos"]) and ca["end"] == cb["end"]
                kerr = (ca["k"].float() - cb["k"].float()).abs().max().item() / cb["k"].float().abs().max().item()
                assert kerr <= tol, (tag, dtype, kerr)
            print(tag, dtype, "ok")
    print("cached mixer ok")
    """)
    assert "cached mixer ok" in out
