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
