"""Routing of the mixer's attention core to the kernels (host logic; the GPU case
at the bottom checks the windowed route against the oracle)."""
import logging
import sys
import types

import numpy as np
import pytest
import torch

from machinelearning_b200 import flash_cuda, mixer_glue


class FakeMixer:
    def __init__(self, **kw):
        self.flash_cuda = True
        self.causal = True
        self.block_attn = 0
        self.swa_window = 0
        self.swa_sinks = 0
        self._flash_declined = False
        self.__dict__.update(kw)


def _cpu_qkv():
    q = torch.zeros(1, 8, 2, 64)
    return q, q.clone(), q.clone()


def test_install_registers_module_and_attribute():
    pkg = types.ModuleType("fakelab")
    sys.modules["fakelab"] = pkg
    try:
        mixer_glue.install("fakelab")
        assert sys.modules["fakelab.flash_cuda"] is flash_cuda
        assert pkg.flash_cuda is flash_cuda
        import importlib
        assert importlib.import_module("fakelab.flash_cuda") is flash_cuda
    finally:
        sys.modules.pop("fakelab", None)
        sys.modules.pop("fakelab.flash_cuda", None)


def test_install_refuses_after_mixers_bound_elsewhere():
    sys.modules["fakelab2"] = types.ModuleType("fakelab2")
    sys.modules["fakelab2.mixers"] = types.ModuleType("fakelab2.mixers")
    sys.modules["fakelab2.flash_cuda"] = types.ModuleType("fakelab2.flash_cuda")
    try:
        with pytest.raises(RuntimeError):
            mixer_glue.install("fakelab2")
    finally:
        for n in ("fakelab2", "fakelab2.mixers", "fakelab2.flash_cuda"):
            sys.modules.pop(n, None)


@pytest.mark.parametrize("kw,needle", [
    (dict(flash_cuda=False), "off"),
    (dict(causal=False, swa_window=8, swa_sinks=2), "causal-only"),      # nanolab/mixers.py:323-325
    (dict(block_attn=16, swa_window=8, swa_sinks=2), "mutually exclusive"),  # mixers.py:300-304
    (dict(swa_window=8, swa_sinks=8), "sinks"),
])
def test_decline_reasons_before_any_load(kw, needle):
    q, k, v = _cpu_qkv()
    why = mixer_glue.decline_reason(FakeMixer(**kw), q, k, v)
    assert why is not None and needle in why


def test_mask_block_follows_the_mixers_mode():
    """``block_attn`` wins (mixers.py:319-321); a non-causal step is one block of the whole sequence."""
    assert mixer_glue.mask_block(FakeMixer(), 100) == 0
    assert mixer_glue.mask_block(FakeMixer(block_attn=16), 100) == 16
    assert mixer_glue.mask_block(FakeMixer(causal=False), 100) == 100
    assert mixer_glue.mask_block(FakeMixer(causal=False, block_attn=8), 100) == 8


def test_cpu_tensors_decline_and_warn_once(caplog):
    q, k, v = _cpu_qkv()
    m = FakeMixer(swa_window=4, swa_sinks=1)
    with caplog.at_level(logging.WARNING, logger="machinelearning_b200.mixer_glue"):
        assert mixer_glue.attention_core(m, q, k, v, 0.125) is None
        assert mixer_glue.attention_core(m, q, k, v, 0.125) is None
    warnings = [r for r in caplog.records if "cannot run" in r.getMessage()]
    assert len(warnings) == 1 and "unsupported inputs" in warnings[0].getMessage()
    assert m._flash_declined


def test_flag_off_is_silent(caplog):
    q, k, v = _cpu_qkv()
    with caplog.at_level(logging.WARNING, logger="machinelearning_b200.mixer_glue"):
        assert mixer_glue.attention_core(FakeMixer(flash_cuda=False), q, k, v, 0.125) is None
    assert not caplog.records


@pytest.mark.gpu
def test_windowed_mixer_routes_through_the_kernel():
    from oracle import attention_f64
    if not flash_cuda.is_available():
        pytest.fail(f"flash_cuda unavailable on a GPU box: {flash_cuda.unavailable_reason()}")
    g = torch.Generator().manual_seed(7)
    B, T, H, Hkv, D = 2, 200, 4, 2, 64
    q = torch.randn(B, T, H, D, generator=g).bfloat16()
    k = torch.randn(B, T, Hkv, D, generator=g).bfloat16()
    v = torch.randn(B, T, Hkv, D, generator=g).bfloat16()
    m = FakeMixer(swa_window=64, swa_sinks=4)
    y = mixer_glue.attention_core(m, q.cuda(), k.cuda(), v.cuda(), 0.125)
    assert y is not None and not m._flash_declined
    ref, _ = attention_f64.attention_fwd(q.double().numpy(), k.double().numpy(), v.double().numpy(),
                                        0.125, window=64, sinks=4)
    err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= 2e-2, err        # relative, bf16 tolerance of the path


@pytest.mark.gpu
@pytest.mark.parametrize("kw,block", [(dict(block_attn=48), 48), (dict(causal=False), 200)])
def test_block_causal_and_bidirectional_steps_route_through_the_kernel(kw, block):
    """The diffusion modes of the mixer (``set_block_attn`` / ``set_causal(False)``, nanolab/model.py:305-314)
    against the oracle with the reference's block-causal mask."""
    from oracle import attention_f64
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    g = torch.Generator().manual_seed(9)
    B, T, H, Hkv, D = 2, 200, 4, 2, 64
    q = torch.randn(B, T, H, D, generator=g).bfloat16()
    k = torch.randn(B, T, Hkv, D, generator=g).bfloat16()
    v = torch.randn(B, T, Hkv, D, generator=g).bfloat16()
    m = FakeMixer(**kw)
    y = mixer_glue.attention_core(m, q.cuda(), k.cuda(), v.cuda(), 0.125)
    assert y is not None and not m._flash_declined
    ref, _ = attention_f64.attention_fwd(q.double().numpy(), k.double().numpy(), v.double().numpy(), 0.125, block=block)
    assert np.abs(y.float().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max()


def _fake_package(name):
    """A stand-in for nanolab: ``<name>.mixers`` bound to this package's ``flash_cuda`` with an ``Attention``
    whose ``forward`` / ``forward_cached`` record their calls."""
    pkg = types.ModuleType(name)
    mixers = types.ModuleType(f"{name}.mixers")
    mixers.flash_cuda = flash_cuda

    class Attention(FakeMixer):
        def forward(self, x, cos, sin, v0=None):
            return ("plain forward", x.shape)

        def forward_cached(self, x, cos, sin, v0, cache, commit, causal=False):
            return ("plain forward_cached", commit, causal)

    mixers.Attention = Attention
    sys.modules[name] = pkg
    sys.modules[f"{name}.mixers"] = mixers
    sys.modules[f"{name}.flash_cuda"] = flash_cuda
    return mixers


def test_fuse_mixer_patches_and_hands_declined_steps_to_the_own_methods():
    """``fuse_mixer`` swaps the class's two methods, ``unfuse_mixer`` restores them, and every step the kernels
    decline before touching the projections (flag off, CPU tensors; for the cached step also gradients being
    recorded or a window without ``causal``) goes to the class's own method with its arguments intact."""
    mixers = _fake_package("fakelab3")
    try:
        own_forward, own_cached = mixers.Attention.forward, mixers.Attention.forward_cached
        mixer_glue.fuse_mixer("fakelab3")
        assert mixers.Attention.forward is mixer_glue.fused_attention_forward
        assert mixers.Attention.forward_cached is mixer_glue.fused_attention_forward_cached
        mixer_glue.fuse_mixer("fakelab3")                                     # idempotent
        x = torch.zeros(2, 8, 16)
        for kw in (dict(flash_cuda=False), dict()):                          # flag off; flag on but CPU tensors
            m = mixers.Attention(**kw)
            assert m.forward(x, None, None) == ("plain forward", x.shape)
            assert m.forward_cached(x, None, None, None, {}, True, causal=True) == ("plain forward_cached", True, True)
        with torch.no_grad():
            m = mixers.Attention(swa_window=8, swa_sinks=2)
            assert m.forward_cached(x, None, None, None, {}, False) == ("plain forward_cached", False, False)
        mixer_glue.unfuse_mixer("fakelab3")
        assert mixers.Attention.forward is own_forward and mixers.Attention.forward_cached is own_cached
        mixer_glue.unfuse_mixer("fakelab3")                                   # nothing left to undo
    finally:
        mixer_glue.unfuse_mixer("fakelab3")
        for n in ("fakelab3", "fakelab3.mixers", "fakelab3.flash_cuda"):
            sys.modules.pop(n, None)


def test_fuse_mixer_refuses_a_package_bound_to_another_module():
    mixers = _fake_package("fakelab4")
    mixers.flash_cuda = types.ModuleType("someone_elses_flash_cuda")
    try:
        with pytest.raises(RuntimeError):
            mixer_glue.fuse_mixer("fakelab4")
    finally:
        for n in ("fakelab4", "fakelab4.mixers", "fakelab4.flash_cuda"):
            sys.modules.pop(n, None)
