"""The C-ABI library on a machine without a GPU: it builds, loads, exports every
declared symbol, and its host-side argument checks answer before any launch."""
import ctypes
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "nlfa.h"


@pytest.fixture(scope="module")
def lib():
    from machinelearning_b200 import _build, _lib
    _build.build()
    return _lib.load()


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(nlfa_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("nlfa_fwd", "nlfa_bwd", "nlfa_bwd_scratch_bytes", "nlfa_selftest",
                 "nlfa_strerror", "nlfa_device_status", "nlfa_resolve_path"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in nlfa.h but not exported"


def test_ctypes_signatures_cover_the_header():
    from machinelearning_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_strerror_and_version(lib):
    assert lib.nlfa_version() >= 1
    assert lib.nlfa_strerror(0) == b"ok"
    for code in range(1, 16):
        assert lib.nlfa_strerror(code) not in (b"", b"ok", b"unknown status")
    assert lib.nlfa_strerror(999) == b"unknown status"


def test_path_resolution_mirrors_use_mma(lib):
    from machinelearning_b200 import _lib as L
    assert lib.nlfa_resolve_path(L.DTYPE_BF16, 64, L.PATH_AUTO) == L.PATH_TENSOR
    assert lib.nlfa_resolve_path(L.DTYPE_F16, 128, L.PATH_AUTO) == L.PATH_TENSOR
    assert lib.nlfa_resolve_path(L.DTYPE_F32, 64, L.PATH_AUTO) == L.PATH_SIMT
    assert lib.nlfa_resolve_path(L.DTYPE_BF16, 32, L.PATH_AUTO) == L.PATH_TENSOR   # zero-padded 64-wide tiles
    assert lib.nlfa_resolve_path(L.DTYPE_F32, 32, L.PATH_AUTO) == L.PATH_SIMT
    assert lib.nlfa_resolve_path(L.DTYPE_BF16, 64, L.PATH_SIMT) == L.PATH_SIMT
    assert lib.nlfa_resolve_path(L.DTYPE_F32, 64, L.PATH_TENSOR) == -7     # use_mma=True on fp32
    assert lib.nlfa_resolve_path(L.DTYPE_BF16, 48, L.PATH_AUTO) == -4
    assert lib.nlfa_resolve_path(7, 64, L.PATH_AUTO) == -3


def test_argument_checks_answer_without_a_gpu(lib):
    from machinelearning_b200 import _lib as L
    one = ctypes.c_void_p(16)       # non-null, aligned; never dereferenced by the checks below
    fwd = lambda **kw: lib.nlfa_fwd(
        kw.get("q", one), one, one, one, one, kw.get("B", 1), kw.get("T", 8), kw.get("H", 2),
        kw.get("Hkv", 1), kw.get("D", 64), 0.125, kw.get("window", 0), kw.get("sinks", 0),
        kw.get("dtype", L.DTYPE_F32), kw.get("path", L.PATH_AUTO), None)
    assert fwd(Hkv=0) == 2 and fwd(H=3, Hkv=2) == 2 and fwd(B=-1) == 2
    assert fwd(dtype=9) == 3
    assert fwd(D=48) == 4
    assert fwd(window=4, sinks=4) == 5 and fwd(window=0, sinks=1) == 5 and fwd(window=-2) == 5
    assert fwd(path=L.PATH_TENSOR) == 7
    assert fwd(B=0) == 0 and fwd(T=0) == 0                 # empty problem: successful no-op
    assert fwd(q=None) == 1
    assert fwd(q=ctypes.c_void_p(24)) == 6                 # not 16-byte aligned
    assert lib.nlfa_bwd_scratch_bytes(2, 100, 4) == 2 * 100 * 4 * 4
    assert lib.nlfa_bwd_scratch_bytes(0, 100, 4) == 0
    bwd = lib.nlfa_bwd(one, one, one, one, one, one, one, one, one, one, 8, 1, 8, 2, 1, 64,
                       0.125, 0, 0, L.DTYPE_F32, L.PATH_AUTO, None)
    assert bwd == 11                                        # scratch too small
    # the one-pass backward: its own scratch size, refusals before anything touches a device
    tape = lib.nlfa_bwd_scratch_bytes(2, 300, 4)
    assert lib.nlfa_bwd_fused_scratch_bytes(2, 300, 4, 128) == (tape + 255) // 256 * 256      # no fused pass at 128
    tiles = 2 * 4 * 3
    assert lib.nlfa_bwd_fused_scratch_bytes(2, 300, 4, 64) == (tape + 255) // 256 * 256 + 256 + tiles * 128 * 64 * 4
    passes = lambda mask, D=64, dtype=L.DTYPE_BF16, path=L.PATH_TENSOR, nbytes=1 << 30: lib.nlfa_bwd_passes(
        one, one, one, one, one, one, one, one, one, one, nbytes, 1, 300, 2, 1, D, 0.125, 0, 0, dtype, path, mask, None)
    assert passes(L.PASS_FUSED | L.PASS_DKV) == 7 and passes(L.PASS_FUSED | L.PASS_DQ) == 7 and passes(16) == 7
    assert passes(L.PASS_FUSED, D=128) == 7                 # tensor-core path, head dims up to 64 only
    assert passes(L.PASS_FUSED, dtype=L.DTYPE_F32, path=L.PATH_AUTO) == 7
    assert passes(L.PASS_FUSED, nbytes=lib.nlfa_bwd_scratch_bytes(1, 300, 2)) == 11
    errs = (ctypes.c_float * 2)()
    assert lib.nlfa_selftest(L.DTYPE_BF16, 64, one, 16, errs, None) == 11
    assert lib.nlfa_selftest(L.DTYPE_F32, 64, one, 1 << 20, errs, None) == 7


@pytest.mark.parametrize("T,window,sinks", [
    (1024, 0, 0), (300, 0, 0), (129, 0, 0),
    (1024, 256, 0), (1024, 64, 4), (900, 300, 130), (700, 256, 0), (2048, 512, 4),
    (300, 400, 4), (511, 64, 0), (640, 129, 128), (384, 128, 0), (385, 1, 0),
])
@pytest.mark.parametrize("stream_rows", [64, 128])
def test_mask_geometry_matches_the_elementwise_predicate(lib, T, window, sinks, stream_rows):
    """Block ranges, fully-visible tests and one-edge classifications against every (q, k) pair."""
    assert lib.nlfa_check_mask_geometry(T, window, sinks, stream_rows) == 0


@pytest.mark.parametrize("T,block", [(1024, 1), (1024, 32), (1024, 96), (1024, 128), (900, 256), (700, 333),
                                     (1024, 4096), (385, 7), (2048, 512)])
@pytest.mark.parametrize("stream_rows", [64, 128])
def test_block_causal_geometry_matches_the_elementwise_predicate(lib, T, block, stream_rows):
    """The same checks for the block-causal mask (keep key k for query q iff q // block >= k // block)."""
    assert lib.nlfa_check_mask_geometry_masked(T, 0, 0, block, stream_rows) == 0
    assert lib.nlfa_check_mask_geometry_masked(T, 64, 4, block, stream_rows) < 0      # a window excludes it


def test_mask_geometry_rejects_bad_arguments(lib):
    assert lib.nlfa_check_mask_geometry(0, 0, 0, 128) < 0
    assert lib.nlfa_check_mask_geometry(256, 8, 8, 128) < 0
    assert lib.nlfa_check_mask_geometry(256, 0, 4, 128) < 0
    assert lib.nlfa_check_mask_geometry(256, 0, 0, 96) < 0


def test_backward_kernel_count_follows_the_layout(lib):
    """``nlfa_bwd_kernel_count``: Delta + dK/dV + dQ; two kernels where the dQ pass forms Delta (head dim
    64, tensor-core path, a large problem -- every problem is large next to the one SM a machine
    without a GPU reports); Delta + pass + convert for the one-pass layout; 0 for what is refused."""
    from machinelearning_b200 import _lib
    count = lib.nlfa_bwd_kernel_count
    bf16, f32 = _lib.DTYPE_BF16, _lib.DTYPE_F32
    tensor, simt = _lib.PATH_TENSOR, _lib.PATH_SIMT
    assert count(32, 1024, 12, 128, bf16, tensor, _lib.PASS_ALL) == 3
    assert count(32, 1024, 12, 32, bf16, tensor, _lib.PASS_ALL) == 3
    assert count(32, 1024, 12, 64, f32, simt, _lib.PASS_ALL) == 3
    assert count(32, 1024, 12, 64, bf16, simt, _lib.PASS_ALL) == 3
    assert count(32, 1024, 12, 64, bf16, tensor, _lib.PASS_DKV) == 1
    assert count(32, 1024, 12, 64, bf16, tensor, _lib.PASS_DELTA | _lib.PASS_DKV) == 2
    assert count(32, 1024, 12, 64, bf16, tensor, _lib.PASS_DELTA | _lib.PASS_FUSED) == 3
    assert count(32, 1024, 12, 64, bf16, tensor, _lib.PASS_FUSED | _lib.PASS_DQ) == 0
    assert count(32, 1024, 12, 128, bf16, tensor, _lib.PASS_FUSED) == 0
    assert count(32, 1024, 12, 64, f32, tensor, _lib.PASS_ALL) == 0
    assert count(0, 1024, 12, 64, bf16, tensor, _lib.PASS_ALL) == 0
    assert count(32, 1024, 12, 64, bf16, tensor, 0) == 0
    # the large-problem layout (needs the device's SM count on a GPU box; 4,096 x 12 x 8 tiles is large anywhere)
    assert count(4096, 1024, 12, 64, bf16, tensor, _lib.PASS_ALL) == 2
    assert count(4096, 1024, 12, 64, bf16, tensor, _lib.PASS_DELTA | _lib.PASS_DQ) == 1
