"""The Python module that mirrors nanolab/flash_cuda.py, on a machine with no GPU."""
import importlib

import pytest
import torch


@pytest.fixture()
def fc():
    from machinelearning_b200 import flash_cuda
    return importlib.reload(flash_cuda)


def test_public_names_match_the_reference_module(fc):
    for name in ("SUPPORTED_HEAD_DIMS", "SUPPORTED_DTYPES", "MMA_DTYPES", "MMA_BWD_HEAD_DIMS",
                 "supports", "effective_dtype", "is_available", "unavailable_reason",
                 "mma_available", "mma_unavailable_reason", "flash_attn", "sdpa_reference", "main"):
        assert hasattr(fc, name), name
    assert fc.SUPPORTED_HEAD_DIMS == (32, 64, 128)
    assert fc.SUPPORTED_DTYPES == (torch.float32, torch.float16, torch.bfloat16)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_unavailable_without_a_device_and_never_falls_back(fc):
    assert fc.is_available() is False
    assert fc.unavailable_reason() == "no CUDA device"
    assert fc.mma_available() is False and fc.mma_unavailable_reason() == "no CUDA device"
    q = torch.randn(1, 8, 2, 64)
    assert fc.supports(q, q, q) is False              # CPU tensors are not supported inputs
    with pytest.raises(ValueError):
        fc.flash_attn(q, q, q)
    with pytest.raises(RuntimeError):                  # the native entry refuses, no CPU path
        fc.fwd(q, q, q, 0.125, False)


def test_env_switch_disables_the_library(fc, monkeypatch):
    monkeypatch.setenv("NANOLAB_FLASH_CUDA", "0")
    assert fc.is_available() is False
    assert fc.unavailable_reason() == "disabled by NANOLAB_FLASH_CUDA=0"


def test_effective_dtype_without_autocast(fc):
    a, b = torch.randn(1, 4, 2, 64), torch.randn(1, 4, 2, 64, dtype=torch.bfloat16)
    assert fc.effective_dtype(a, a, a) is torch.float32
    assert fc.effective_dtype(a, a, b) is None


def test_supports_shape_rules(fc):
    class Fake:
        """A stand-in with the tensor attributes supports() reads, claiming to be on CUDA."""
        def __init__(self, shape, dtype=torch.bfloat16):
            self.shape, self.dtype, self.is_cuda = torch.Size(shape), dtype, True
        def dim(self):
            return len(self.shape)
    ok = (Fake((2, 16, 4, 64)), Fake((2, 16, 2, 64)), Fake((2, 16, 2, 64)))
    fc_eff = fc.effective_dtype
    fc.effective_dtype = lambda q, k, v: q.dtype if q.dtype == k.dtype == v.dtype else None
    try:
        assert fc.supports(*ok)
        assert not fc.supports(Fake((2, 16, 4, 48)), Fake((2, 16, 2, 48)), Fake((2, 16, 2, 48)))
        assert not fc.supports(Fake((2, 16, 4, 64)), Fake((2, 16, 3, 64)), Fake((2, 16, 3, 64)))
        assert not fc.supports(Fake((2, 16, 4, 64)), Fake((2, 15, 2, 64)), Fake((2, 15, 2, 64)))
        assert not fc.supports(Fake((16, 4, 64)), Fake((16, 2, 64)), Fake((16, 2, 64)))
        assert not fc.supports(Fake((2, 16, 4, 64), torch.float64), Fake((2, 16, 2, 64), torch.float64),
                               Fake((2, 16, 2, 64), torch.float64))
        assert not fc.supports(Fake((2, 16, 4, 64)), Fake((2, 16, 0, 64)), Fake((2, 16, 0, 64)))
    finally:
        fc.effective_dtype = fc_eff


@pytest.mark.parametrize("w,s", [(0, 1), (4, 4), (4, 5), (-1, 0)])
def test_window_refusals_match_the_mixer(fc, w, s):
    with pytest.raises(ValueError):
        fc.check_window(w, s)


def test_window_accepts_valid(fc):
    fc.check_window(0, 0)
    fc.check_window(64, 4)
    fc.check_window(1, 0)
