"""Scheduler counters under concurrency: a captured graph replaying on one stream while eager
launches run on another (needs a B200).

The persistent kernels take their work units from a pair of device counters.  A launch made under
stream capture keeps the counters it was given for as long as its graph is replayed, so those come
from a range that is never handed to another launch; eager launches take turns on a ring of their
own.  Two kernels that shared a pair would skip units and leave rows unwritten, silently -- the
check is bit-equality with results computed alone.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graph_replay_and_eager_launches_do_not_share_work_counters():
    from machinelearning_b200 import flash_cuda as fc
    assert fc.mma_available(), fc.mma_unavailable_reason()
    torch.manual_seed(11)
    D = 64
    scale = 1.0 / math.sqrt(D)
    mk = lambda b, t, h: torch.randn(b, t, h, D, device="cuda").bfloat16()
    qa, ka, va, da = mk(2, 512, 4), mk(2, 512, 2), mk(2, 512, 2), mk(2, 512, 4)     # the graph's problem
    qb, kb, vb, db = mk(3, 384, 2), mk(3, 384, 2), mk(3, 384, 2), mk(3, 384, 2)     # the eager one

    def run(q, k, v, d):
        o, lse = fc.fwd(q, k, v, scale, True)
        return (o, lse, *fc.bwd(d, q, k, v, o, lse, scale, True))

    want_a = [t.clone() for t in run(qa, ka, va, da)]
    want_b = [t.clone() for t in run(qb, kb, vb, db)]
    torch.cuda.synchronize()

    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        run(qa, ka, va, da)                      # warm-up on the capture stream
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            got_a = run(qa, ka, va, da)
    torch.cuda.synchronize()

    bad = 0
    for i in range(1000):
        with torch.cuda.stream(side):
            graph.replay()
        got_b = run(qb, kb, vb, db)              # eager, on the default stream, overlapping the replay
        if i % 50 == 49:
            torch.cuda.synchronize()
            bad += sum(not torch.equal(g, w) for g, w in zip(got_a, want_a))
            bad += sum(not torch.equal(g, w) for g, w in zip(got_b, want_b))
    torch.cuda.synchronize()
    assert bad == 0


def test_overlapped_launches_give_the_bits_of_serialised_ones():
    """The tensor-core kernels are launched with programmatic stream serialization (a kernel's set-up
    runs beside its predecessor's last CTAs, the dQ pass fills the SMs the dK/dV pass leaves);
    ``NLFA_PDL=0`` launches them the plain way.  The two must agree bit for bit, back to back, with a
    window and without."""
    import os
    import subprocess
    import sys
    import pathlib
    root = pathlib.Path(__file__).resolve().parent.parent
    script = f"""
import sys, math, hashlib
sys.path.insert(0, {str(root)!r})
import torch
from machinelearning_b200 import flash_cuda as fc
assert fc.mma_available(), fc.mma_unavailable_reason()
h = hashlib.sha256()
for (B, T, H, Hkv, D, w, s) in ((3, 700, 4, 2, 64, 0, 0), (2, 1024, 4, 4, 128, 0, 0), (2, 900, 4, 2, 64, 128, 4)):
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda heads: torch.randn(B, T, heads, D, device="cuda", generator=g).bfloat16()
    q, k, v, d = mk(H), mk(Hkv), mk(Hkv), mk(H)
    for _ in range(20):                        # back to back: every launch has a predecessor still running
        o, lse = fc.fwd(q, k, v, 1 / math.sqrt(D), True, w, s)
        grads = fc.bwd(d, q, k, v, o, lse, 1 / math.sqrt(D), True, w, s)
    torch.cuda.synchronize()
    for t in (o, lse, *grads):
        h.update(t.cpu().contiguous().view(torch.uint8).numpy().tobytes())
print("digest", h.hexdigest())
"""
    digests = []
    for flag in ("1", "0"):
        env = dict(os.environ, NLFA_PDL=flag)
        r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
        digests.append(r.stdout.strip().splitlines()[-1])
    assert digests[0] == digests[1]


def test_delta_formed_in_the_dq_pass_gives_the_bits_of_the_delta_kernel():
    """Large problems at head dim 64 skip the Delta kernel: the dQ pass forms the row sums of dO * O
    itself (same additions in the same order) and runs before the dK/dV pass.  ``NLFA_DELTA_IN_DQ``
    forces either layout; every gradient must agree bit for bit, causal, windowed and block-causal,
    with query rows past the end of the last tile."""
    import os
    import subprocess
    import sys
    import pathlib
    root = pathlib.Path(__file__).resolve().parent.parent
    script = f"""
import sys, math, hashlib
sys.path.insert(0, {str(root)!r})
import torch
from machinelearning_b200 import flash_cuda as fc
assert fc.mma_available(), fc.mma_unavailable_reason()
h = hashlib.sha256()
for (B, T, H, Hkv, w, s, blk) in ((3, 700, 4, 2, 0, 0, 0), (2, 1000, 6, 6, 128, 4, 0), (2, 517, 4, 1, 0, 0, 96), (40, 1024, 12, 12, 0, 0, 0)):
    g = torch.Generator(device="cuda").manual_seed(6)
    mk = lambda heads: torch.randn(B, T, heads, 64, device="cuda", generator=g).bfloat16()
    q, k, v, d = mk(H), mk(Hkv), mk(Hkv), mk(H)
    for _ in range(3):
        o, lse = fc.fwd(q, k, v, 0.125, True, w, s, blk)
        grads = fc.bwd(d, q, k, v, o, lse, 0.125, True, w, s, block=blk)
    torch.cuda.synchronize()
    for t in grads:
        h.update(t.cpu().contiguous().view(torch.uint8).numpy().tobytes())
print("digest", h.hexdigest())
"""
    digests = []
    for flag in ("1", "0"):
        env = dict(os.environ, NLFA_DELTA_IN_DQ=flag)
        r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
        digests.append(r.stdout.strip().splitlines()[-1])
    assert digests[0] == digests[1]
