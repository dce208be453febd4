"""The whole-model caller against nanolab's own GPT (fixture written from nanolab by
``tests/golden/make_whole_model_golden.py``), its data-parallel step over two gloo
ranks on CPU, and -- on the GPU -- the same fixture with the attention core routed
through the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from machinelearning_b200 import whole_model as wm

from conftest import GOLDEN

FIXTURE = GOLDEN / "whole_model_tiny.npz"
TINY = dict(n_layer=2, d_model=32, n_head=4, n_kv_head=2, head_dim=32, block_size=40, vocab_size=61)
CASES = {"causal": {}, "swa": dict(swa_window=16, swa_sinks=2)}


def _load(tag, device="cpu", **extra):
    d = np.load(FIXTURE)
    model = wm.GPT(wm.ModelShape(**TINY, **CASES[tag], **extra))
    state = {k.split("/param/")[1]: torch.from_numpy(d[k]) for k in d.files if k.startswith(f"{tag}/param/")}
    state["lm_head.weight"] = state["tok_emb.weight"]
    model.load_state_dict(state, strict=True)
    model.to(device)
    grads = {k.split("/grad/")[1]: d[k] for k in d.files if k.startswith(f"{tag}/grad/")}
    idx, tgt = torch.from_numpy(d[f"{tag}/idx"]).to(device), torch.from_numpy(d[f"{tag}/tgt"]).to(device)
    return model, idx, tgt, float(d[f"{tag}/loss"]), d[f"{tag}/logits"], grads


def _check(model, idx, tgt, loss_ref, logits_ref, grads_ref, tol):
    logits, loss = model(idx, tgt)
    loss.backward()
    assert abs(loss.item() - loss_ref) <= tol
    assert np.abs(logits.detach().cpu().numpy() - logits_ref).max() <= tol
    got = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
    assert set(got) == set(grads_ref)          # e.g. layer 0's vr_lambda has none, as in nanolab
    for n, g in got.items():
        ref = grads_ref[n]
        assert np.abs(g.cpu().numpy() - ref).max() <= tol * max(1.0, np.abs(ref).max()), n


@pytest.mark.parametrize("tag", list(CASES))
def test_caller_matches_nanolab_gpt_on_cpu(tag):
    model, *rest = _load(tag)
    _check(model, *rest, tol=2e-6)


def test_phase1_shape_has_nanolabs_parameter_count():
    s = wm.ModelShape()
    attn = 4 * s.d_model * s.d_model + 2 * s.head_dim + (s.d_model + 1) * s.n_head + 1
    block = attn + 3 * s.d_model * s.ffn_hidden + 2 * s.d_model
    total = s.vocab_size * s.d_model + s.d_model + s.n_layer * block      # tied embedding + final norm
    assert total == 123_699_612 and s.ffn_hidden == 2048


def test_flag_on_cpu_tensors_declines_to_sdpa_once(caplog):
    model, idx, tgt, loss_ref, *_ = _load("causal", flash_cuda=True)
    with caplog.at_level("WARNING"):
        _, loss = model(idx, tgt)
    assert abs(loss.item() - loss_ref) <= 2e-6
    assert sum("flash_cuda=True but the kernel cannot run" in r.message for r in caplog.records) == TINY["n_layer"]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(3)
        model = wm.GPT(wm.ModelShape(**TINY, zero_init_proj=False))
        x, y = wm.synthetic_tokens(TINY["vocab_size"], 4, TINY["block_size"], seed=5)
        lo, hi = rank * 2, rank * 2 + 2
        step = wm.DataParallelStep(model, dtype=torch.float32, bucket_mb=1)
        step.bucket_elems = 20_000                      # several buckets on this tiny model
        for _ in range(2):
            step.step(x[lo:hi], y[lo:hi])
        assert step.collectives >= 4
        if rank == 0:
            torch.save({n: p.detach() for n, p in model.named_parameters()}, out)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_equal_one_rank_on_the_whole_batch(tmp_path):
    out = tmp_path / "dp.pt"
    mp.spawn(_dp_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    torch.manual_seed(3)
    model = wm.GPT(wm.ModelShape(**TINY, zero_init_proj=False))
    x, y = wm.synthetic_tokens(TINY["vocab_size"], 4, TINY["block_size"], seed=5)
    step = wm.DataParallelStep(model, dtype=torch.float32)
    for _ in range(2):
        step.step(x, y)
    dp = torch.load(out)
    for n, p in model.named_parameters():
        assert torch.allclose(p.detach(), dp[n], atol=2e-6, rtol=0), n


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True], ids=["torch-passes", "fused-prologue-epilogue"])
@pytest.mark.parametrize("tag", list(CASES))
def test_caller_through_the_kernels_matches_nanolab_gpt(tag, fused):
    """fp32 tensors, ``flash_cuda=True``: every layer's core runs in the library (D=32, GQA 4/2), with
    QK-norm, RoPE, value blend and head gate as torch passes or as the fused kernels."""
    from machinelearning_b200 import flash_cuda
    assert flash_cuda.is_available(), flash_cuda.unavailable_reason()
    model, *rest = _load(tag, device="cuda", flash_cuda=True, fused_prologue=fused, fused_epilogue=fused)
    calls = []
    real = flash_cuda.flash_attn
    try:
        flash_cuda.flash_attn = lambda *a, **k: (calls.append(k), real(*a, **k))[1]
        _check(model, *rest, tol=2e-5)
    finally:
        flash_cuda.flash_attn = real
    assert len(calls) == TINY["n_layer"]
    assert all(c["window"] == CASES[tag].get("swa_window", 0) for c in calls)


@pytest.mark.gpu
def test_bf16_autocast_step_runs_the_tensor_core_path_and_lowers_the_loss():
    torch.manual_seed(0)
    shape = wm.ModelShape(n_layer=2, d_model=256, n_head=4, head_dim=64, block_size=256, vocab_size=512,
                          flash_cuda=True)
    model = wm.GPT(shape).cuda()
    x, y = (t.cuda() for t in wm.synthetic_tokens(512, 8, 256, seed=1))
    step = wm.DataParallelStep(model, lr=3e-4)
    losses = [step.step(x, y).item() for _ in range(12)]
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]
    assert not any(b.mixer._flash_declined for b in model.blocks)


@pytest.mark.gpu
def test_fused_and_separate_passes_agree_under_bf16_autocast():
    """Same weights, same tokens, bf16 autocast: loss and gradients with the prologue, value-blend and
    gate kernels against the torch passes they replace (2e-2 relative, ``max|a - b| / max|b|``)."""
    shape = dict(n_layer=2, d_model=256, n_head=4, n_kv_head=2, head_dim=64, block_size=256, vocab_size=512,
                 flash_cuda=True, zero_init_proj=False)
    x, y = (t.cuda() for t in wm.synthetic_tokens(512, 4, 256, seed=2))
    out = []
    for fused in (False, True):
        torch.manual_seed(1)
        model = wm.GPT(wm.ModelShape(**shape, fused_prologue=fused, fused_epilogue=fused)).cuda()
        with torch.no_grad():
            for b in model.blocks:
                b.mixer.q_norm.weight.add_(0.2 * torch.randn_like(b.mixer.q_norm.weight))
                b.mixer.gate.weight.normal_(0.0, 0.05)
                b.mixer.vr_lambda.fill_(0.3)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = model(x, y)
        loss.backward()
        out.append((loss.item(), {n: p.grad.float() for n, p in model.named_parameters() if p.grad is not None}))
    (l0, g0), (l1, g1) = out
    assert abs(l0 - l1) <= 2e-3 * abs(l0)
    assert set(g0) == set(g1)
    for n in g0:
        assert (g0[n] - g1[n]).abs().max().item() <= 2e-2 * g0[n].abs().max().item() + 1e-6, n


@pytest.mark.gpu
def test_captured_step_follows_the_eager_trajectory():
    """The whole step replayed from a CUDA graph against the same steps issued eagerly: same weights, same
    batches; the losses agree step by step (bf16 autocast; the kernels are bit-reproducible, torch's own
    reductions may differ in the last place between the two)."""
    shape = dict(n_layer=2, d_model=256, n_head=4, head_dim=64, block_size=256, vocab_size=512, flash_cuda=True,
                 zero_init_proj=False)
    batches = [tuple(t.cuda() for t in wm.synthetic_tokens(512, 4, 256, seed=s)) for s in range(5)]
    runs = []
    for captured in (False, True):
        torch.manual_seed(2)
        model = wm.GPT(wm.ModelShape(**shape)).cuda()
        step = wm.DataParallelStep(model, lr=3e-4)
        if captured:
            step.capture(*batches[0])
        runs.append([step.step(x, y).item() for x, y in batches])
    eager, graph = runs
    assert all(np.isfinite(eager)) and all(np.isfinite(graph))
    assert max(abs(a - b) for a, b in zip(eager, graph)) <= 2e-3 * max(eager)
    assert graph[0] != graph[-1]                      # the replays do train
