"""Forward + backward of batches that live in host memory.

The attention path is independent per batch element (``sharding.py``), so a
host-resident batch does not have to be copied in whole before the first kernel
starts: it is cut into batch slices, and three CUDA streams carry, at the same
time, the host-to-device copy of slice ``i + 1``, the kernels of slice ``i``
(``flash_cuda.fwd`` and ``flash_cuda.bwd``, the native entries behind
``flash_attn`` and its autograd backward) and the device-to-host copy of slice
``i - 1``.
PCIe is full duplex, so a step costs about the larger of the two copy times
instead of the sum of both copies and the kernels.

There is no counterpart in the reference: its callers hold device tensors
(``nanolab/mixers.py:347-370``).  Results are bit-identical to one whole-batch
call, because every kernel treats batch elements independently.
"""
from __future__ import annotations

import math

import torch

from . import flash_cuda, sharding


class HostPipeline:
    """Reusable streams, events and device staging for one problem shape.

    ``run`` reads pinned host tensors ``q [B,T,H,D]``, ``k, v [B,T,Hkv,D]``,
    ``dout [B,T,H,D]`` and fills pinned host tensors ``o, dq [B,T,H,D]`` and
    ``dk, dv [B,T,Hkv,D]``.  The inputs must be complete in host memory when ``run``
    is called (they are read by a stream of the pipeline's own, not the caller's).
    Everything is asynchronous with respect to the host; the caller's current
    stream is made to wait for the last copy out, so ordinary stream semantics
    (events, ``synchronize``) apply to the results.

    ``n_slices``: two measured best for calls that follow one another (a 201 MB
    step each way: 4.58 ms against 4.79 with one slice and 5.11 with eight;
    consecutive calls overlap anyway, and finer slices interleave the two PCIe
    directions more finely, which slows both); a single isolated call gains
    from more slices, since only they overlap its own copies with its kernels.
    """

    def __init__(self, q_shape, kv_shape, dtype, device, n_slices: int = 2):
        B = q_shape[0]
        if kv_shape[0] != B:
            raise ValueError("q and k/v must share the batch dimension")
        self.device = torch.device(device)
        self.n_slices = max(1, min(int(n_slices), B))
        self.bounds = [sharding.split_range(B, self.n_slices, i) for i in range(self.n_slices)]
        with torch.cuda.device(self.device):
            self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream() for _ in range(3))
            # device staging for the whole batch: slices never alias, so the only reuse
            # hazard is between consecutive calls, handled by the per-slice events below
            self.dq_in = torch.empty(q_shape, dtype=dtype, device=self.device)
            self.dk_in = torch.empty(kv_shape, dtype=dtype, device=self.device)
            self.dv_in = torch.empty(kv_shape, dtype=dtype, device=self.device)
            self.ddo_in = torch.empty(q_shape, dtype=dtype, device=self.device)
            self.ev_in = [torch.cuda.Event() for _ in range(self.n_slices)]
            self.ev_cmp = [torch.cuda.Event() for _ in range(self.n_slices)]
            self.used = False

    def run(self, q, k, v, dout, o, dq, dk, dv, scale=None, window: int = 0, sinks: int = 0):
        for t in (q, k, v, dout, o, dq, dk, dv):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("HostPipeline.run takes pinned host tensors")
        if scale is None:
            scale = 1.0 / math.sqrt(q.shape[-1])
        if not flash_cuda.supports(self.dq_in, self.dk_in, self.dv_in) or not flash_cuda.is_available():
            raise RuntimeError(f"flash_cuda cannot run these inputs ({flash_cuda.unavailable_reason()})")
        flash_cuda.check_window(window, sinks)
        use_mma = flash_cuda._tensor_path_fits(q.dtype, q.shape[-1]) and flash_cuda.mma_available()
        cur = torch.cuda.current_stream(self.device)
        # The inputs are host memory, complete when this is called, so the copy-in stream does
        # not wait for the caller's stream: the next call's copies in then overlap this call's
        # copies out.  (Reuse of the device staging is ordered by the per-slice events.)
        self.s_out.wait_stream(cur)
        keep = []      # outputs of the compute stream, alive until the copy stream is done with them
        for i, (b0, b1) in enumerate(self.bounds):
            sl = slice(b0, b1)
            with torch.cuda.stream(self.s_in):
                if self.used:
                    self.s_in.wait_event(self.ev_cmp[i])      # previous call's kernels on this slice
                self.dq_in[sl].copy_(q[sl], non_blocking=True)
                self.dk_in[sl].copy_(k[sl], non_blocking=True)
                self.dv_in[sl].copy_(v[sl], non_blocking=True)
                self.ddo_in[sl].copy_(dout[sl], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[i])
                qs, ks, vs = self.dq_in[sl], self.dk_in[sl], self.dv_in[sl]
                # the two native entries behind flash_attn and its autograd backward, called
                # directly: no graph is needed when both directions run back to back
                y, lse = flash_cuda.fwd(qs, ks, vs, scale, use_mma, window, sinks)
                grads = flash_cuda.bwd(self.ddo_in[sl], qs, ks, vs, y, lse, scale, use_mma, window, sinks)
                self.ev_cmp[i].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_cmp[i])
                for dst, src in zip((o, dq, dk, dv), (y, *grads)):
                    dst[sl].copy_(src, non_blocking=True)
                keep.append((y, grads))
        self.used = True
        cur.wait_stream(self.s_out)
        # The outputs were allocated on the compute stream.  Their memory goes back to that
        # stream's pool when `keep` is dropped, so the stream is first made to wait for the
        # copies that read them (cheaper than per-tensor record_stream, which keeps blocks out
        # of the pool until an event query and sends the allocator back to cudaMalloc).
        self.s_cmp.wait_stream(self.s_out)
        del keep
