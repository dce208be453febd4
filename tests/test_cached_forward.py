"""The KV-cached block forward: the oracle against what nanolab's own ``forward_hidden_window`` fed to
and got from SDPA (``tests/golden/cached_forward.npz``), host-side argument checks, and -- on the GPU --
the kernel against the same recorded calls and against the oracle at a decode-sized shape."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import cached_f64

D_ = np.load(GOLDEN / "cached_forward.npz")
CALLS = sorted({k.rsplit("/", 1)[0] for k in D_.files})


def _call(name):
    causal, window, sinks = (int(x) for x in D_[name + "/meta"])
    return dict(q=D_[name + "/q"], k=D_[name + "/k"], v=D_[name + "/v"], y=D_[name + "/y"], mask=D_[name + "/mask"],
                qpos=D_[name + "/qpos"], kpos=D_[name + "/kpos"], scale=float(D_[name + "/scale"]),
                causal=bool(causal), window=window, sinks=sinks)


@pytest.mark.parametrize("name", CALLS)
def test_oracle_reproduces_nanolabs_masks_and_sdpa_results(name):
    c = _call(name)
    keep = cached_f64.keep_mask(c["qpos"], c["kpos"], c["causal"], c["window"], c["sinks"])
    assert np.array_equal(keep, c["mask"])
    y, _ = cached_f64.forward(c["q"], c["k"], c["v"], c["scale"], c["qpos"], c["kpos"], c["causal"], c["window"],
                              c["sinks"])
    assert np.abs(y - c["y"]).max() <= 1e-12


def test_fixture_covers_eviction():
    gaps = [n for n in CALLS if n.startswith("swa") and np.any(np.diff(D_[n + "/kpos"]) > 1)]
    assert gaps, "no recorded call has non-contiguous key positions"


def test_entry_point_refuses_bad_arguments_before_any_launch():
    from machinelearning_b200 import _build, _lib
    _build.build()
    f = _lib.load().nlfa_fwd_cached
    args = lambda **kw: [kw.get("q", 16), 16, 16, 16, None, None, None, kw.get("B", 1), kw.get("T", 4), kw.get("H", 4),
                         kw.get("Hkv", 2), kw.get("L", 8), kw.get("D", 64), 0.125, kw.get("causal", 1),
                         kw.get("window", 0), kw.get("sinks", 0), kw.get("dtype", 2), None, 0, None]
    assert f(*args(D=48)) == 4
    assert f(*args(dtype=7)) == 3
    assert f(*args(Hkv=3)) == 2
    assert f(*args(window=4, sinks=4)) == 5
    assert f(*args(window=4, causal=0)) == 5          # a window needs a causal block
    assert f(*args(T=9, L=8)) == 2                    # contiguous default: the block is part of the keys
    assert f(*args(q=None)) == 1
    assert f(*args(B=0)) == 0
    sb = _lib.load().nlfa_fwd_cached_scratch_bytes
    assert sb(8, 32, 12, 4, 1056, 64) == 0                      # enough row chunks: no split
    assert sb(1, 64, 16, 16, 16448, 128) == 64 * 16 * 3 * 129 * 4      # three splits of a long cache


def test_python_wrapper_rejects_cpu_tensors_and_bidirectional_windows():
    from machinelearning_b200 import flash_cuda
    q, k = torch.zeros(1, 4, 2, 64), torch.zeros(1, 1, 8, 64)
    with pytest.raises(ValueError):
        flash_cuda.flash_attn_cached(q, k, k)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", CALLS)
def test_kernel_matches_nanolabs_recorded_calls(name, dtype):
    """fp32: max-abs 1e-5 against SDPA's float64 result; bf16: 2e-2 relative against the oracle on the
    same rounded inputs (``max|x - ref| / max|ref|``)."""
    from machinelearning_b200 import flash_cuda
    c = _call(name)
    t = lambda a: torch.from_numpy(a).to("cuda", dtype)
    q, k, v = t(c["q"]), t(c["k"]), t(c["v"])
    y, lse = flash_cuda.flash_attn_cached(q, k, v, c["scale"], qpos=torch.from_numpy(c["qpos"]),
                                          kpos=torch.from_numpy(c["kpos"]), causal=c["causal"], window=c["window"],
                                          sinks=c["sinks"], return_lse=True)
    if dtype == torch.float32:
        assert np.abs(y.double().cpu().numpy() - c["y"]).max() <= 1e-5
    ref, lse_ref = cached_f64.forward(q.double().cpu().numpy(), k.double().cpu().numpy(), v.double().cpu().numpy(),
                                      c["scale"], c["qpos"], c["kpos"], c["causal"], c["window"], c["sinks"])
    tol = 1e-5 if dtype == torch.float32 else 2e-2 * np.abs(ref).max()
    assert np.abs(y.double().cpu().numpy() - ref).max() <= tol
    assert np.abs(lse.double().cpu().numpy() - lse_ref).max() <= (1e-5 if dtype == torch.float32 else 1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("D", [32, 64, 128])
def test_decode_sized_block_with_default_positions_and_an_unseen_row(D):
    """A 32-token block over 1,000 cached keys, GQA 8/2, contiguous default positions, against the oracle;
    and a window case whose explicit positions leave one query row with no visible key (zeros, -inf)."""
    from machinelearning_b200 import flash_cuda
    g = torch.Generator().manual_seed(D)
    B, T, H, Hkv, L = 2, 32, 8, 2, 1032
    q = torch.randn(B, T, H, D, generator=g).bfloat16().cuda()
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16().cuda()
    v = torch.randn(B, Hkv, L, D, generator=g).bfloat16().cuda()
    for causal, window, sinks in ((False, 0, 0), (True, 0, 0), (True, 200, 4)):
        y = flash_cuda.flash_attn_cached(q, k, v, causal=causal, window=window, sinks=sinks)
        ref, _ = cached_f64.forward(q.double().cpu().numpy(), k.double().cpu().numpy(), v.double().cpu().numpy(),
                                    1.0 / np.sqrt(D), np.arange(L - T, L), np.arange(L), causal, window, sinks)
        assert np.abs(y.double().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max()
    qpos = torch.tensor([5] + list(range(L - T + 1, L)))           # row 0 sits before every key it could reach
    kpos = torch.arange(100, 100 + L)
    y, lse = flash_cuda.flash_attn_cached(q, k, v, qpos=qpos, kpos=kpos, causal=True, window=64, sinks=0,
                                          return_lse=True)
    assert torch.count_nonzero(y[:, 0]).item() == 0 and torch.isinf(lse[:, :, 0]).all()
    assert torch.isfinite(y.float()).all()


@pytest.mark.gpu
def test_key_split_and_single_walk_agree():
    """A long cache with few query rows takes the key split (scratch given); without scratch one CTA walks
    all keys.  Same rows either way, up to fp32 rounding of the combination."""
    from machinelearning_b200 import _lib, flash_cuda
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    lib = _lib.load()
    B, T, H, Hkv, L, D = 1, 16, 4, 2, 4000, 64
    nbytes = lib.nlfa_fwd_cached_scratch_bytes(B, T, H, Hkv, L, D)
    assert nbytes > 0
    g = torch.Generator().manual_seed(1)
    q = torch.randn(B, T, H, D, generator=g).bfloat16().cuda()
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16().cuda()
    v = torch.randn(B, Hkv, L, D, generator=g).bfloat16().cuda()
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    outs = []
    for ptr, size in ((scratch.data_ptr(), nbytes), (None, 0)):
        o = torch.empty_like(q)
        lse = torch.empty(B, H, T, device="cuda")
        st = lib.nlfa_fwd_cached(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), None, None,
                                 B, T, H, Hkv, L, D, 0.125, 1, 0, 0, _lib.DTYPE_BF16, ptr, size,
                                 torch.cuda.current_stream().cuda_stream)
        assert st == 0
        outs.append((o.float(), lse))
    (o1, l1), (o2, l2) = outs
    assert (o1 - o2).abs().max().item() <= 1e-2 * o2.abs().max().item()
    assert (l1 - l2).abs().max().item() <= 1e-4
    ref, lse_ref = cached_f64.forward(q.double().cpu().numpy(), k.double().cpu().numpy(), v.double().cpu().numpy(),
                                      0.125, np.arange(L - T, L), np.arange(L), True)
    assert np.abs(o1.double().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max()
    assert np.abs(l1.double().cpu().numpy() - lse_ref).max() <= 1e-3


TC_SHAPES = [
    # B, T, H, Hkv, L, D, causal, window, sinks, explicit positions with gaps
    (8, 32, 12, 4, 1056, 64, True, 0, 0, False),
    (8, 32, 12, 12, 1056, 64, False, 0, 0, False),       # a bidirectional block, MHA
    (8, 16, 12, 4, 4112, 64, True, 0, 0, False),
    (8, 32, 12, 4, 288, 64, True, 256, 4, False),
    (1, 64, 16, 16, 16448, 128, True, 0, 0, False),      # few rows, a long cache: the keys are split over CTAs
    (2, 48, 8, 2, 700, 32, True, 0, 0, False),           # head dim 32 on 64-wide tiles; 4 heads x 32 positions per tile
    (2, 40, 6, 2, 900, 64, True, 300, 8, True),          # positions after eviction: not contiguous
    (1, 200, 4, 4, 600, 128, True, 0, 0, True),          # more than one query tile per KV head
]


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,H,Hkv,L,D,causal,window,sinks,gaps", TC_SHAPES)
def test_tensor_core_kernel_matches_oracle_and_the_fp32_kernel(B, T, H, Hkv, L, D, causal, window, sinks, gaps):
    """The tcgen05 form of the cached block forward (forced with ``use_mma=True``) against the float64
    oracle (2e-2 relative on bf16, LSE 1e-3) and against the fp32 kernel on the same inputs."""
    from machinelearning_b200 import flash_cuda
    assert flash_cuda.mma_available(), flash_cuda.mma_unavailable_reason()
    g = torch.Generator().manual_seed(L + D)
    q = torch.randn(B, T, H, D, generator=g).bfloat16().cuda()
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16().cuda()
    v = torch.randn(B, Hkv, L, D, generator=g).bfloat16().cuda()
    if gaps:                                     # keys keep their order but skip positions; the block comes last
        kpos_np = np.cumsum(1 + (np.arange(L) % 7 == 0)).astype(np.int64)
        qpos_np = kpos_np[L - T:].copy()
        qpos, kpos = torch.from_numpy(qpos_np), torch.from_numpy(kpos_np)
    else:
        qpos = kpos = None
        qpos_np, kpos_np = np.arange(L - T, L), np.arange(L)
    kw = dict(qpos=qpos, kpos=kpos, causal=causal, window=window, sinks=sinks, return_lse=True)
    y, lse = flash_cuda.flash_attn_cached(q, k, v, use_mma=True, **kw)
    y32, lse32 = flash_cuda.flash_attn_cached(q, k, v, use_mma=False, **kw)
    auto, _ = flash_cuda.flash_attn_cached(q, k, v, **kw)
    assert torch.equal(auto, y)                  # every shape here is one the library takes the tensor cores for
    sub = slice(0, min(B, 2))                    # the oracle materialises [T, L] per head: two batch elements suffice
    ref, lse_ref = cached_f64.forward(q[sub].double().cpu().numpy(), k[sub].double().cpu().numpy(),
                                      v[sub].double().cpu().numpy(), 1.0 / np.sqrt(D), qpos_np, kpos_np, causal,
                                      window, sinks)
    assert np.abs(y[sub].double().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max()
    assert np.abs(lse[sub].double().cpu().numpy() - lse_ref).max() <= 1e-3
    assert (y.float() - y32.float()).abs().max().item() <= 2e-2 * y32.float().abs().max().item()
    assert (lse - lse32).abs().max().item() <= 1e-3


@pytest.mark.gpu
def test_tensor_core_kernel_is_refused_where_it_does_not_apply():
    from machinelearning_b200 import flash_cuda
    q = torch.randn(1, 4, 2, 64, device="cuda").bfloat16()           # 4 rows per KV head, 40 keys: fp32 kernel territory
    k = torch.randn(1, 2, 40, 64, device="cuda").bfloat16()
    with pytest.raises(ValueError, match="does not apply"):
        flash_cuda.flash_attn_cached(q, k, k, use_mma=True)
    assert torch.isfinite(flash_cuda.flash_attn_cached(q, k, k).float()).all()
