"""Attention forward+backward throughput on B200, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

A step is one forward plus one backward of the causal bf16 attention path over
one batch of synthetic input (B=32, H=12, T=1024, D=64, scale 1/8: the nanolab
124M-model shape).  With N ranks that batch is partitioned (``sharding.plan``:
32 / N batch elements per GPU, no exchange step in the path: strong scaling);
after the timed region the shards of O, LSE, dQ, dK and dV are gathered over
NCCL and compared, bit for bit, with rank 0's own run of the whole batch.  The
figure for N full batches on N GPUs (weak scaling) rides along as ``weak``.

Prints one JSON line:
  value      whole-job TFLOP/s, algorithmic FLOPs (2 forward + 5 backward GEMMs
             over the unmasked pairs), inputs resident in HBM, CUDA-event time,
             slowest rank
  e2e        the same metric for pinned host buffers through
             ``host_pipeline.HostPipeline`` (``flash_cuda.fwd`` + ``flash_cuda.bwd``
             per batch slice, three streams): host->device copies of q, k, v, dO
             and device->host copies of O, dQ, dK, dV inside the timed region
  roofline   the dominant kernel timed alone against the measured dense bf16 peak
  cpu_baseline  the reference's CPU attention (torch SDPA + autograd, restated in
             oracle/sdpa_port.py) on this box's host cores, bounded sample

``--impl reference`` times only that CPU path, on the same config and metric.

``--workload c4`` is the other half of the metric: tokens/s of the whole nanolab
GPT training step (12 layers, d_model 768, 12x64 heads, context 1024, global
batch 64 sequences split over the ranks, gradient all-reduce over NCCL) with the
attention core in the library, next to the same step with the flag off (SDPA).
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (B, T, H, Hkv, D, window, sinks): the whole job's shape; N GPUs split B
    "c2": (32, 1024, 12, 12, 64, 0, 0),
    "c3": (16, 4096, 16, 16, 64, 256, 0),
    "c5": (8, 16384, 16, 16, 128, 0, 0),
}
WORKLOAD_TEXT = {
    "c2": "causal bf16 attention fwd+bwd, B=32 H=12 T=1024 D=64, scale 1/8",
    "c3": "sliding-window bf16 attention fwd+bwd, B=16 H=16 T=4096 D=64 window=256",
    "c5": "long-context causal bf16 attention fwd+bwd, B=8 H=16 T=16384 D=128, scale 1/sqrt(128)",
}
ALGORITHMIC_BYTES_PER_ELEMENT = 2      # every tensor of the path is bf16; LSE and Delta are fp32 rows
WHOLE_MODEL = "c4"
WHOLE_MODEL_TEXT = ("nanolab GPT training step, flash_cuda on: 12 layers d_model=768 12x64 heads RoPE RMSNorm "
                    "QK-norm SwiGLU(2048) vocab=50304 context=1024, global batch 64 sequences, bf16 autocast, "
                    "AdamW (stands in for nanolab's Muon+AdamW)")
METRIC = "attention fwd+bwd TFLOP/s (bf16 causal)"
METRIC_TOKENS = "nanolab tokens/sec (whole-model training step)"
FALLBACK_PEAK_TFLOPS = 1590.0
E2E_SLICES = 2


def pairs(T, window, sinks):
    if window == 0:
        return T * (T + 1) // 2
    span = window - sinks
    total = 0
    for q in range(T):
        lo = max(0, q - span + 1)
        total += (q - lo + 1) + min(sinks, lo)
    return total


def flops(B, T, H, D, window, sinks):
    """(forward, backward) algorithmic FLOPs: 2 and 5 GEMMs over the unmasked pairs."""
    n = pairs(T, window, sinks)
    return 4.0 * D * n * B * H, 10.0 * D * n * B * H


def measured_hbm():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"])
    except Exception:                                             # noqa: BLE001
        return 6650.0


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
        except Exception:                                         # noqa: BLE001
            pass
    return FALLBACK_PEAK_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(shape, seed, device, pin=False):
    """q, k, v, dO ~ N(0,1) generated in fp32 from a seed, then cast to bf16."""
    B, T, H, Hkv, D, _, _ = shape
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for heads in (H, Hkv, Hkv, H):
        t = torch.randn(B, T, heads, D, generator=g, dtype=torch.float32).to(torch.bfloat16)
        if pin:
            out.append(t.pin_memory())          # stays on the host, page-locked
        else:
            out.append(t if device == "cpu" else t.to(device))
    return out


# ----------------------------------------------------------------------------
# CPU arm: the reference's own attention path on host cores
# ----------------------------------------------------------------------------

def cpu_sample_batch(shape):
    """Batch elements of the workload one CPU step covers (a bounded sample: seconds, not minutes)."""
    B, T = shape[0], shape[1]
    return 1 if T > 8192 else max(1, B // 4)


def cpu_fwd_bwd_tflops(shape, reps, warmup):
    """The reference's CPU attention (``oracle/sdpa_port.py``: torch SDPA + autograd, the chunked
    window path for SWA) on all host cores, over a sample of the batch: median of ``reps`` timed
    forward+backward runs after ``warmup`` untimed ones.  Both arms measure it this way."""
    from oracle import sdpa_port            # test infrastructure: only timed here, never shipped
    B, T, H, Hkv, D, window, sinks = shape
    sb = cpu_sample_batch(shape)
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, do = make_inputs((sb, T, H, Hkv, D, window, sinks), 1234, "cpu")
    scale = 1.0 / math.sqrt(D)
    times = []
    for i in range(warmup + reps):
        t0 = time.perf_counter()
        sdpa_port.cpu_fwd_bwd(q, k, v, do, scale, window, sinks)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    ff, fb = flops(sb, T, H, D, window, sinks)
    sec = statistics.median(times)
    return (ff + fb) / sec / 1e12, sec, sb


def cpu_baseline_record(shape, reps, warmup):
    tf, sec, sb = cpu_fwd_bwd_tflops(shape, reps, warmup)
    sample = (f"{sb} of {shape[0]} batch elements per step, torch CPU SDPA + autograd in bf16 "
              f"(oracle/sdpa_port.py), {warmup} warm-up + {reps} timed steps, median {sec:.3f} s")
    return {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": sample}, sec, sb


def run_reference_arm(args, shape, rank, world):
    if rank != 0:
        return
    B = shape[0]
    cpu, sec, sb = cpu_baseline_record(shape, reps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3 * B / sb, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[args.workload]},
        "cpu_sample": {"what": cpu["sample"], "ms_per_step": "sample time scaled by B / sample size"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

class Step:
    """Pre-allocated buffers and direct C-ABI calls for one forward+backward."""

    def __init__(self, shape, q, k, v, do):
        from machinelearning_b200 import _lib, flash_cuda
        if not flash_cuda.is_available():
            raise RuntimeError(f"libnlfa unavailable: {flash_cuda.unavailable_reason()}")
        if not flash_cuda.mma_available():
            raise RuntimeError(f"tensor-core path unavailable: {flash_cuda.mma_unavailable_reason()}")
        self.L, self.lib = _lib, _lib.load()
        self.B, self.T, self.H, self.Hkv, self.D, self.window, self.sinks = shape
        self.scale = 1.0 / math.sqrt(self.D)
        self.q, self.k, self.v, self.do = q, k, v, do
        self.o = torch.empty_like(q)
        self.lse = torch.empty(self.B, self.H, self.T, dtype=torch.float32, device=q.device)
        self.dq, self.dk, self.dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        self.scratch = torch.empty(self.lib.nlfa_bwd_fused_scratch_bytes(self.B, self.T, self.H, self.D),
                                   dtype=torch.uint8, device=q.device)

    def _dims(self):
        return (self.B, self.T, self.H, self.Hkv, self.D, self.scale, self.window, self.sinks,
                self.L.DTYPE_BF16, self.L.PATH_TENSOR)

    def fwd(self):
        st = self.lib.nlfa_fwd(self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                               self.o.data_ptr(), self.lse.data_ptr(), *self._dims(),
                               torch.cuda.current_stream().cuda_stream)
        self.L.check("nlfa_fwd", st)

    def bwd(self, passes=7):
        st = self.lib.nlfa_bwd_passes(
            self.do.data_ptr(), self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
            self.o.data_ptr(), self.lse.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(),
            self.dv.data_ptr(), self.scratch.data_ptr(), self.scratch.numel(), *self._dims(),
            passes, torch.cuda.current_stream().cuda_stream)
        self.L.check("nlfa_bwd_passes", st)

    def step(self):
        self.fwd()
        self.bwd()

    def outputs(self):
        return {"o": self.o, "lse": self.lse, "dq": self.dq, "dk": self.dk, "dv": self.dv}

    @property
    def launches_per_step(self):
        """Forward + what the backward launches for this shape: Delta, dK/dV, dQ -- or, for a large
        problem at D = 64, the dQ pass that forms Delta itself and then dK/dV."""
        return 1 + self.lib.nlfa_bwd_kernel_count(self.B, self.T, self.H, self.D, self.L.DTYPE_BF16,
                                                  self.L.PATH_TENSOR, self.L.PASS_ALL)

    def captured(self):
        """The same step as one CUDA graph (replayed, the host issues one launch per step)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            self.step()                         # attributes and tensor maps are set up outside the capture
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                self.step()
        torch.cuda.current_stream().wait_stream(side)
        return graph


def time_region(fn, iters):
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def kernel_times(step: Step, iters=10):
    """Average device time of each kernel, timed alone with CUDA events on its stream."""
    L = step.L
    out = {}
    names = [("fwd", step.fwd), ("delta", lambda: step.bwd(L.PASS_DELTA)),
             ("dkv", lambda: step.bwd(L.PASS_DKV)), ("dq", lambda: step.bwd(L.PASS_DQ))]
    if step.launches_per_step == 3:
        names.append(("dq_forming_delta", lambda: step.bwd(L.PASS_DELTA | L.PASS_DQ)))   # what the step runs
    if step.D <= 64:
        names.append(("one_pass_bwd", lambda: step.bwd(L.PASS_FUSED)))     # the alternative layout, for the record
    for name, fn in names:
        for _ in range(3):
            fn()
        out[name] = time_region(fn, iters)
    return out


def dram_traffic(kernel, workload):
    path = ROOT / "profiles" / "dram_traffic.json"
    if path.exists():
        try:
            return json.loads(path.read_text()).get(f"{kernel}:{workload}")
        except Exception:                                         # noqa: BLE001
            return None
    return None


def algorithmic_bytes(B, T, H, Hkv, D):
    """(forward, backward) bytes that have to move: every input and output once, plus the fp32 rows."""
    qo, kv, rows = B * T * H * D * 2, B * T * Hkv * D * 2, B * H * T * 4
    fwd = 2 * qo + 2 * kv + rows                            # q, o, k, v, lse
    bwd = 4 * qo + 4 * kv + 4 * rows                        # q, o, dO, dq, k, v, dk, dv, lse, Delta written, read twice
    return fwd, bwd


def other_workload(name, dev, iters=5):
    """Kernel-only forward+backward of another named shape (whole batch on this GPU), CUDA events."""
    shape = WORKLOADS[name]
    B, T, H, Hkv, D, window, sinks = shape
    q, k, v, do = make_inputs(shape, 4321, dev)
    step = Step(shape, q, k, v, do)
    for _ in range(3):
        step.step()
    ms = time_region(step.step, iters)
    ff, fb = flops(B, T, H, D, window, sinks)
    bf, bb = algorithmic_bytes(B, T, H, Hkv, D)
    rec = {"workload": WORKLOAD_TEXT[name], "ms_per_step": ms, "tflops": (ff + fb) / (ms * 1e-3) / 1e12,
           "algorithmic_gb_per_s": (bf + bb) / (ms * 1e-3) / 1e9, "iters": iters}
    del step, q, k, v, do
    torch.cuda.empty_cache()
    return rec


def same_box_comparison(shape, dev, iters=20):
    """The public call a user makes -- ``flash_attn`` + autograd -- next to torch's SDPA (what nanolab's
    mixer runs with the flag off) on the same inputs and GPU: forward and forward + backward, both as
    calls back to back between two events (throughput) and as the median of calls timed one at a time
    with a synchronisation each (what the reference's self-check prints, ``flash_cuda.py:297-312``).
    Plain causal shapes only (``sdpa_reference`` is the causal arm)."""
    from machinelearning_b200 import flash_cuda
    B, T, H, Hkv, D, window, sinks = shape
    q, k, v, do = make_inputs(shape, 77, dev)
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    scale = 1.0 / math.sqrt(D)
    arms = {"these_kernels": lambda: flash_cuda.flash_attn(q, k, v, scale),
            "torch_sdpa": lambda: flash_cuda.sdpa_reference(q, k, v, scale)}
    out = {"what": "flash_attn / SDPA through autograd on resident inputs, ms; back_to_back = calls queued between "
                   "two events, per_call = median of calls synchronised one at a time", "iters": iters}
    for name, fwd in arms.items():
        both = lambda fwd=fwd: torch.autograd.grad(fwd(), (q, k, v), do)
        for _ in range(5):
            both()
        out[name] = {"back_to_back": {"fwd": time_region(fwd, iters), "fwd_bwd": time_region(both, iters)},
                     "per_call": {"fwd": flash_cuda._median_ms(fwd, iters), "fwd_bwd": flash_cuda._median_ms(both, iters)}}
    del q, k, v, do
    torch.cuda.empty_cache()
    return out


def run_gpu_arm(args, shape, rank, world, local_rank):
    import torch.distributed as dist
    from machinelearning_b200 import flash_cuda, host_pipeline, sharding

    B, T, H, Hkv, D, window, sinks = shape
    if B % world:
        raise SystemExit(f"batch {B} does not split over {world} ranks")
    # the CPU baseline first, before this process has started any CUDA work: the same measurement the
    # reference arm makes (rank 0, one GPU only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, _, _ = cpu_baseline_record(shape, reps=5, warmup=2)

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # every rank draws the whole job's inputs from the same seed and keeps its share: what the
    # ranks compute together is then exactly what one GPU computes alone
    gq, gk, gv, gdo = make_inputs(shape, 1000, "cpu")
    plan = sharding.plan(B, Hkv, world, rank)
    hq, hk, hv, hdo = (t.contiguous() for t in sharding.take_shard(gq, gk, gv, gdo, plan))
    local_shape = (hq.shape[0], T, hq.shape[2], hk.shape[2], D, window, sinks)
    q, k, v, do = (t.to(dev) for t in (hq, hk, hv, hdo))
    step = Step(local_shape, q, k, v, do)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- kernel-only throughput, inputs resident in HBM.  One GPU: eager launches (a step is
    # hundreds of microseconds, the host keeps ahead).  Several GPUs: the per-GPU share shrinks to
    # tens of microseconds, so the step is replayed from a CUDA graph -- the GPU is timed, not Python.
    graph = step.captured() if world > 1 else None
    run = graph.replay if graph is not None else step.step
    warm = max(args.warmup, 3)
    for _ in range(warm):
        run()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.__enter__()
    # Timing hygiene: a per-GPU working set that fits the 126 MB L2 (the named batch split 4 or 8
    # ways) would be served from L2 step after step, so L2 is flushed between timed steps and every
    # step gets an event pair of its own, outside which the flush runs.  The flush overwrites a
    # 256 MB buffer and then reads another one, so that the timed step starts on a cold L2 without
    # also paying for the write-back of the flush's dirty lines.  These steps are launched eagerly:
    # the host enqueues a step's kernels while the flush in front of them is still running, so the
    # events bracket GPU time only (a graph launch inside the bracket would add its own latency).
    # Larger working sets evict themselves and are timed as one region.
    working_set = 8 * q.numel() * q.element_size()
    cold = working_set < 1.5 * 126e6
    if not cold:
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            run()
        end.record()
        barrier()
        ms_local = start.elapsed_time(end) / args.steps
    else:
        dirty = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        clean = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
        pairs_ = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                  for _ in range(args.steps)]
        for first, last in pairs_:
            dirty.zero_()
            clean.max()
            first.record()
            step.step()
            last.record()
        barrier()
        ms_local = sum(first.elapsed_time(last) for first, last in pairs_) / args.steps
        del dirty, clean
    # keep the GPU busy a little longer so the clock sampler sees load even for short runs
    if sampler:
        t_end = time.time() + 1.0
        while time.time() < t_end:
            run()
        torch.cuda.synchronize()
        sampler.__exit__(None, None, None)
    ms = sharding.max_over_ranks(ms_local, dev)
    ff, fb = flops(B, T, H, D, window, sinks)               # the whole job's
    value = (ff + fb) / (ms * 1e-3) / 1e12

    # ---- several GPUs: the shards gathered over NCCL against one GPU's run of the whole batch
    verified = None
    eager_ms = None
    weak = None
    if world > 1:
        eager_ms = sharding.max_over_ranks(time_region(step.step, args.steps), dev)
        warm_graph_ms = sharding.max_over_ranks(time_region(graph.replay, args.steps), dev) if cold else None
        step.step()
        torch.cuda.synchronize()
        gathered = {n: sharding.gather_batch_shards(t, B) for n, t in step.outputs().items()}
        if rank == 0:
            full = Step(shape, *(t.to(dev) for t in (gq, gk, gv, gdo)))
            full.step()
            torch.cuda.synchronize()
            verified = {n: bool(torch.equal(gathered[n], t)) for n, t in full.outputs().items()}
            del full
        del gathered
        torch.cuda.empty_cache()
        barrier()
        # weak scaling beside it: every rank a whole batch of its own, no graph needed at that size
        wq, wk, wv, wdo = make_inputs(shape, 2000 + rank, dev)
        wstep = Step(shape, wq, wk, wv, wdo)
        for _ in range(3):
            wstep.step()
        barrier()
        wms = sharding.max_over_ranks(time_region(wstep.step, args.steps), dev)
        weak = {"value": world * (ff + fb) / (wms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": wms,
                "global_batch": B * world}
        del wstep, wq, wk, wv, wdo
        torch.cuda.empty_cache()
        barrier()

    # ---- end to end through the public API, host buffers, copies inside the timed region
    hq, hk, hv, hdo = (t.pin_memory() for t in (hq, hk, hv, hdo))
    host_out = [torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv)]
    scale = 1.0 / math.sqrt(D)
    # batch slices: copy-in, kernels and copy-out of neighbouring slices -- and of consecutive steps --
    # overlap.  Two slices measured best over consecutive steps (4.58 ms against 4.79 with one and
    # 5.11 with eight on the same box; both PCIe directions flat out take 4.3 ms).
    pipe = host_pipeline.HostPipeline(tuple(hq.shape), tuple(hk.shape), hq.dtype, dev, n_slices=E2E_SLICES)

    def e2e_step():
        pipe.run(hq, hk, hv, hdo, *host_out, scale=scale, window=window, sinks=sinks)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_iters = max(3, min(args.steps, 10))
    e2e_ms = sharding.max_over_ranks(time_region(e2e_step, e2e_iters), dev)
    barrier()
    e2e_value = (ff + fb) / (e2e_ms * 1e-3) / 1e12
    h2d = world * sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = world * sum(t.numel() * t.element_size() for t in host_out)

    if rank != 0:
        return
    # ---- per-kernel times and the roofline of the dominant one (rank 0, kernels timed alone)
    kt = kernel_times(step)
    # FLOPs per launch on this rank's share.  Algorithmic: the backward's 5 GEMMs are S, dP, dV, dK
    # (dK/dV kernel) and dQ (dQ kernel); the dQ kernel's own S and dP are recomputation and are not
    # counted.  Executed counts them (what the tensor pipe actually ran).
    gemm = 2.0 * D * pairs(T, window, sinks) * local_shape[0] * H
    kflops = {"fwd": 2 * gemm, "dkv": 4 * gemm, "dq": 1 * gemm}
    kexec = {"fwd": 2 * gemm, "dkv": 4 * gemm, "dq": 3 * gemm}
    dominant = max(("fwd", "dkv", "dq"), key=lambda n: kt[n])
    peak, peak_src = measured_peak()
    achieved = kflops[dominant] / (kt[dominant] * 1e-3) / 1e12
    clocks = sampler.summary() if sampler else None
    traffic = dram_traffic(dominant, args.workload) if world == 1 else None

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[args.workload], "global_batch": B,
                   "per_gpu_batch": local_shape[0],
                   "parallelism": f"batch split over {world} GPU(s) (sharding.plan), no collective in the path",
                   "timing": ("eager launches, every step between an event pair of its own, enqueued while the L2 "
                              "flush in front of it runs" if cold else
                              f"CUDA graph replay of forward+backward ({step.launches_per_step} kernels) between two events"
                              if graph is not None else "eager launches between two events"),
                   "l2": "working set (q,k,v,o,dO,dq,dk,dv) larger than the 126 MB L2"
                         if not cold else
                         f"per-GPU working set {working_set / 1e6:.0f} MB (the named shape, split): L2 flushed between "
                         "timed steps (256 MB overwritten, then 256 MB read), one CUDA-event pair per step",
                   "flops_per_step": ff + fb},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "pipeline": f"{E2E_SLICES} batch slices per GPU; copy-in, kernels and copy-out on three streams"},
        "gpu_launches": step.launches_per_step * args.steps,
        "kernel_ms": kt,
        "roofline": {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_src,
                     "flops_per_launch": kflops[dominant],
                     "executed_tflops": kexec[dominant] / (kt[dominant] * 1e-3) / 1e12,
                     "traffic": traffic,
                     "traffic_source": "ncu capture of this kernel on this workload (profiles/dram_traffic.json), "
                                       "not measured by this run"},
        "frac_of_peak_fwd_bwd": value / world / peak,
        "clocks": clocks,
    }
    if world > 1:
        line["verified_against_single_gpu"] = verified
        line["eager_ms_per_step"] = eager_ms            # eager launches, back to back, L2 not flushed
        if warm_graph_ms is not None:
            line["graph_replay_ms_per_step_l2_warm"] = warm_graph_ms     # the same step from L2, for comparison
        line["weak"] = weak
    else:
        others = {}
        for name in ("c3", "c5"):
            if name != args.workload and not args.no_other_workloads:
                others[name] = other_workload(name, dev)
        if "c3" in others:
            others["c3"]["frac_of_hbm_peak"] = others["c3"]["algorithmic_gb_per_s"] / measured_hbm()
        if others:
            line["other_workloads"] = others
        if window == 0 and not args.no_other_workloads:
            line["same_box_comparison"] = same_box_comparison(local_shape, dev)
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# Whole-model arm: tokens/s of the GPT training step that calls the path
# ----------------------------------------------------------------------------

GLOBAL_BATCH = 64


def whole_model_cpu_tokens_per_s(n_seq, reps, warmup=1):
    """The same training step on the host cores (flag off: the mixer's SDPA branch), n_seq sequences."""
    from machinelearning_b200 import whole_model as wm
    torch.set_num_threads(os.cpu_count() or 1)
    torch.manual_seed(0)
    model = wm.GPT(wm.ModelShape(flash_cuda=False))
    step = wm.DataParallelStep(model)
    x, y = wm.synthetic_tokens(model.shape.vocab_size, n_seq, model.shape.block_size, seed=0)
    times = []
    for i in range(warmup + reps):
        t0 = time.perf_counter()
        step.step(x, y)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return n_seq * model.shape.block_size / sec, sec


def run_whole_model_reference_arm(args, rank):
    if rank != 0:
        return
    n_seq = 2
    reps = max(1, min(args.steps, 5))              # a step of the sample is seconds of host time
    tok_s, sec = whole_model_cpu_tokens_per_s(n_seq, reps=reps, warmup=1)
    sample = (f"{n_seq} of {GLOBAL_BATCH} sequences per step on the host cores, attention through torch SDPA "
              f"(the mixer's own branch), bf16 autocast, median of {reps} timed steps of {sec:.2f} s after 1 warm-up")
    line = {
        "impl": "reference", "metric": METRIC_TOKENS, "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3 * GLOBAL_BATCH / n_seq, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WHOLE_MODEL_TEXT.replace("flash_cuda on", "flash_cuda off, CPU"),
                   "global_batch": GLOBAL_BATCH, "cpu_sample": sample},
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def nanolab_own_bench(batch):
    """nanolab's own ``bench_gpu.bench`` (``nanolab/bench_gpu.py:41-110``: its GPT, Muon + AdamW, eager
    launches, wall clock), unmodified, with this package injected as ``nanolab.flash_cuda`` -- flag on,
    flag off, and flag on with ``mixer_glue.fuse_mixer()`` (the mixer's elementwise passes fused as well).  Runs in a child process (``nanolab.mixers`` binds the module at import time); needs the staged
    copy of the reference's caller (``oracle/build_ref.py``) and answers why not when it is absent."""
    code = f"""
import sys, json
sys.path.insert(0, {str(ROOT)!r})
from oracle import build_ref
if not build_ref.nanolab_on_path():
    print(json.dumps({{"unavailable": "the reference's nanolab package is not staged (python oracle/build_ref.py)"}}))
    raise SystemExit(0)
import torch
from machinelearning_b200 import mixer_glue, flash_cuda
mixer_glue.install()
from nanolab import bench_gpu, mixers
from nanolab.config import build_config
assert mixers.flash_cuda is flash_cuda
torch.backends.cuda.matmul.allow_tf32 = True
out = {{"caller": "nanolab", "what": "nanolab.bench_gpu.bench(cfg), phase1 preset, batch {batch} x 1024, bf16, "
       "Muon + AdamW, eager, 5 warm-up + 20 timed steps, wall clock"}}
calls = {{"n": 0}}
real = flash_cuda.fwd
def counted(*a, **k):
    calls["n"] += 1
    return real(*a, **k)
flash_cuda.fwd = counted
for arm, flag, fused in (("flash_cuda_on", True, False), ("flash_cuda_off", False, False),
                        ("flash_cuda_on_fused_mixer", True, True)):
    if fused:       # Attention.forward through the prologue, blend, core and gate kernels (mixer_glue.fuse_mixer)
        mixer_glue.fuse_mixer()
    cfg = build_config("phase1", dict(run_name="bench", batch_size={batch}, block_size=1024, grad_accum=1,
                                      flash_cuda=flag, compile=False, dtype="bf16"))
    calls["n"] = 0
    r = bench_gpu.bench(cfg, peak_flops=1.0)
    out[arm] = {{
        "tokens_per_s": r["tok_s"], "ms_per_step": r["ms_per_step"], "fwd_ms": r["fwd_ms"], "bwd_ms": r["bwd_ms"],
        "opt_ms": r["opt_ms"], "loss": r["loss"], "library_forward_calls": calls["n"]}}
    torch.cuda.empty_cache()
print(json.dumps(out))
"""
    try:
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900)
        if r.returncode != 0:
            return {"unavailable": f"child exited {r.returncode}: {r.stderr.strip().splitlines()[-1:]}"}
        return json.loads(r.stdout.strip().splitlines()[-1])
    except Exception as e:                                        # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}


def run_whole_model_arm(args, rank, world, local_rank):
    import torch.distributed as dist
    from machinelearning_b200 import flash_cuda, qk_prologue, sharding, value_gate, whole_model as wm

    if GLOBAL_BATCH % world:
        raise SystemExit(f"global batch {GLOBAL_BATCH} does not split over {world} ranks")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not flash_cuda.is_available():
        raise SystemExit("attention library unavailable: " + str(flash_cuda.unavailable_reason()))
    per_rank = GLOBAL_BATCH // world
    lo = rank * per_rank

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def build(flag):
        torch.manual_seed(0)                       # same weights on every rank
        model = wm.GPT(wm.ModelShape(flash_cuda=flag)).to(dev)
        return model, wm.DataParallelStep(model)

    # counts the library's launches: 1 forward + 3 backward kernels per flash_attn call, 1 forward +
    # 2 backward kernels (gradient pass, fixed-order reduction) per qk_prologue and per value_blend
    # call, 1 + 1 per head_gate call
    calls = {"n": 0, "prologue": 0, "blend": 0, "gate": 0}
    real_fwd, real_prologue = flash_cuda.fwd, qk_prologue.qk_prologue
    real_blend, real_gate = value_gate.value_blend, value_gate.head_gate

    def counted_blend(*a, **k):
        calls["blend"] += 1
        return real_blend(*a, **k)

    def counted_gate(*a, **k):
        calls["gate"] += 1
        return real_gate(*a, **k)
    value_gate.value_blend, value_gate.head_gate = counted_blend, counted_gate

    def counted_fwd(*a, **k):
        calls["n"] += 1
        return real_fwd(*a, **k)

    def counted_prologue(*a, **k):
        calls["prologue"] += 1
        return real_prologue(*a, **k)
    flash_cuda.fwd = counted_fwd
    qk_prologue.qk_prologue = counted_prologue

    captured = {}
    x_host, y_host = wm.synthetic_tokens(50304, GLOBAL_BATCH, 1024, seed=0)
    x_pin, y_pin = x_host[lo:lo + per_rank].pin_memory(), y_host[lo:lo + per_rank].pin_memory()
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def measure(flag, steps, warmup, sample_clocks):
        model, step = build(flag)
        x, y = x_pin.to(dev), y_pin.to(dev)
        # Same weights and tokens in both arms.  The output projections start at zero, so the first
        # step's loss cannot tell the kernels from SDPA; the loss after three optimiser steps can.
        for key in calls:
            calls[key] = 0
        losses = [step.step(x, y).item() for _ in range(4)]        # the fourth loss has seen three updates
        eager_calls = {key: n // 4 for key, n in calls.items()}       # per step, counted while launching eagerly
        first_loss, third_loss = losses[0], losses[3]
        captured[flag] = False
        if not args.no_graph:
            try:                                   # the whole step as one CUDA graph (both arms alike)
                step.capture(x, y)
                captured[flag] = True
            except Exception as e:                 # noqa: BLE001
                print(f"[bench] step not captured ({type(e).__name__}: {e}); launching eagerly", file=sys.stderr)
                raise
        for _ in range(warmup - 1):
            step.step(x, y)
        barrier()
        sampler = ClockSampler(local_rank) if (rank == 0 and sample_clocks) else None
        if sampler:
            sampler.__enter__()
        resident = time_region(lambda: step.step(x, y), steps)
        n_calls = {key: n * steps for key, n in eager_calls.items()}   # a replayed graph makes no Python calls
        if sampler:
            sampler.__exit__(None, None, None)
        barrier()

        def host_step():                          # token ids from pinned host memory, loss back to the host
            xs, ys = x_pin.to(dev, non_blocking=True), y_pin.to(dev, non_blocking=True)
            loss_host.copy_(step.step(xs, ys), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        host_step()
        barrier()
        e2e = time_region(host_step, max(3, min(steps, 10)))
        barrier()
        loss = (first_loss, third_loss)
        flops_tok = model.flops_per_token()
        step.close()
        del model, step
        gc.collect()
        torch.cuda.empty_cache()
        return (sharding.max_over_ranks(resident, dev), sharding.max_over_ranks(e2e, dev), n_calls, loss,
                flops_tok, sampler.summary() if sampler else None)

    steps, warmup = args.steps, max(args.warmup, 3)
    ms, e2e_ms, n_calls, loss, flops_tok, clocks = measure(True, steps, warmup, True)
    sdpa_ms, sdpa_e2e_ms, _, sdpa_loss, _, _ = measure(False, max(3, steps // 2), 3, False)
    if rank != 0:
        return
    tokens = GLOBAL_BATCH * 1024
    peak, peak_src = measured_peak()
    tok_s = tokens / (ms * 1e-3)
    from machinelearning_b200 import _lib
    attn_bwd_kernels = _lib.load().nlfa_bwd_kernel_count(per_rank, 1024, 12, 64, _lib.DTYPE_BF16, _lib.PATH_TENSOR,
                                                         _lib.PASS_ALL)
    line = {
        "metric": METRIC_TOKENS, "value": tok_s, "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WHOLE_MODEL_TEXT, "global_batch": GLOBAL_BATCH, "per_gpu_batch": per_rank,
                   "parallelism": f"data-parallel x{world}, bucketed NCCL all-reduce of the gradients overlapped with the backward",
                   "l2": "activations and weights far larger than the 126 MB L2",
                   "params": 123699612, "flops_per_token": flops_tok,
                   "launch": "whole step replayed from one CUDA graph" if captured.get(True) else "eager launches"},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 2 * x_pin.numel() * x_pin.element_size(), "d2h_bytes_per_step": 4},
        # per flash_attn call: the forward and the backward's kernels for this per-GPU shape (three, or two
        # when the dQ pass forms Delta itself); the prologue, blend and gate calls launch 3, 3 and 2 each
        "gpu_launches": (1 + attn_bwd_kernels) * n_calls["n"] + 3 * n_calls["prologue"] + 3 * n_calls["blend"]
                        + 2 * n_calls["gate"],
        "library_calls_per_step": {"flash_attn": n_calls["n"] // steps, "qk_prologue": n_calls["prologue"] // steps,
                                   "value_blend": n_calls["blend"] // steps, "head_gate": n_calls["gate"] // steps},
        "model_flops_utilisation": flops_tok * tok_s / world / 1e12 / peak,
        "peak_source": peak_src,
        "first_step_loss": loss[0], "loss_after_3_steps": loss[1],
        "flag_off_sdpa": {"tokens_per_s": tokens / (sdpa_ms * 1e-3), "ms_per_step": sdpa_ms,
                          "first_step_loss": sdpa_loss[0], "loss_after_3_steps": sdpa_loss[1]},
        "flag_on_off_loss_rel_diff_after_3_steps": abs(loss[1] - sdpa_loss[1]) / abs(sdpa_loss[1]),
        "clocks": clocks,
    }
    if world == 1:
        line["nanolab_bench_gpu"] = nanolab_own_bench(GLOBAL_BATCH)
    if world == 1 and not args.no_cpu_baseline:
        cpu_tok_s, sec = whole_model_cpu_tokens_per_s(2, reps=2)
        line["cpu_baseline"] = {"value": cpu_tok_s, "unit": "tokens/s", "cores": torch.get_num_threads(),
                                "kind": "port",
                                "sample": f"2 of {GLOBAL_BATCH} sequences per step on the host cores, flag off "
                                          f"(SDPA), median of 2 steps of {sec:.2f} s"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + [WHOLE_MODEL])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true", help="skip the c3 / c5 kernel-only figures")
    ap.add_argument("--no-graph", action="store_true", help="c4: launch the step eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    shape = WORKLOADS.get(args.workload)

    if args.impl == "reference":
        if args.workload == WHOLE_MODEL:
            run_whole_model_reference_arm(args, rank)
        else:
            run_reference_arm(args, shape, rank, world)
        return 0

    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == WHOLE_MODEL:
            run_whole_model_arm(args, rank, world, local_rank)
        else:
            run_gpu_arm(args, shape, rank, world, local_rank)
    finally:
        if world > 1:
            torch.cuda.synchronize()
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
