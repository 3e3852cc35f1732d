"""Forward + backward for callers whose tensors live in (pinned) host memory.

The batch x head slices of the attention are independent, so a step over host-resident
``q, k, v, dO`` is cut into chunks of (batch, head) slices and pipelined over three CUDA
streams: while chunk ``i`` is computed, chunk ``i+1`` is copied host->device and the
results of chunk ``i-1`` are copied device->host.  PCIe is full duplex, so the step costs
about max(H2D, D2H, compute) instead of their sum, plus one chunk's copy at either end (a
tapered chunk schedule that shrinks those ends was measured and changes nothing: 52.1
against 52.3 ms for a single synchronised run).  Device staging buffers are allocated
once per pipeline object and reused.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .tiled_swa import swa_backward, swa_backward_rot, swa_forward, swa_forward_rot


class HostPipeline:
    """``HostPipeline(device, chunk_slices)``; call ``run`` once per step.

    ``run(q, k, v, do, outs, rope, window, sm_scale)``: ``q, k [1, S, N, d_qk]``, ``v, do [1, S, N, d_v]``
    pinned host tensors (``S`` = batch*head slices), ``outs = (o, dq, dk, dv)`` pinned host
    tensors that receive the results (``do``/gradient outputs may be ``None`` for forward
    only).  ``rope`` is ``None`` or device tensors ``(idx, row_cs, col_cs)``; ``window`` =
    ``(b_size, t_height, t_width, row_size, col_size)``.  Returns after all copies have been
    enqueued; synchronise ``self.done`` (or the device) before reading ``outs`` or changing the
    inputs.  Work queued on the current stream afterwards is not ordered after the copy-out (make
    it ``wait_event(self.done)`` if it must be); consecutive runs overlap: the next run's copy-in
    proceeds while this run's results still travel to the host.
    """

    def __init__(self, device, chunk_slices: int = 32, n_buffers: int = 3):
        self.device = torch.device(device)
        self.chunk = chunk_slices
        self.nbuf = n_buffers
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.done = torch.cuda.Event()
        self._stage = None
        self._buf_free = None      # per staging buffer: event after the last kernel that read it (kept ACROSS runs)

    def _staging(self, shapes, dtype):
        key = (tuple(shapes), dtype)
        if self._stage is None or self._stage[0] != key:
            bufs = [[torch.empty(s, dtype=dtype, device=self.device) for s in shapes] for _ in range(self.nbuf)]
            self._stage = (key, bufs)
            self._buf_free = [None] * self.nbuf
        return self._stage[1]

    def run(self, q, k, v, do, outs: Sequence[Optional[torch.Tensor]], rope, window, sm_scale):
        S = q.shape[1]
        c = min(self.chunk, S)
        with_bwd = do is not None
        ins = (q, k, v, do) if with_bwd else (q, k, v)
        shapes = [(1, c) + tuple(t.shape[2:]) for t in ins]
        stage = self._staging(shapes, q.dtype)
        compute = torch.cuda.current_stream(self.device)
        in_ready = [torch.cuda.Event() for _ in range(self.nbuf)]
        # A run may start while the kernels of the previous run still read the staging buffers (nothing else orders
        # the copy-in stream after them): the "buffer is free" events therefore live on the object, not in the call.
        buf_free = self._buf_free
        out_events = []
        n_chunks = (S + c - 1) // c
        for i in range(n_chunks):
            lo, hi = i * c, min(S, (i + 1) * c)
            n = hi - lo
            b = i % self.nbuf
            with torch.cuda.stream(self.s_in):
                if buf_free[b] is not None:
                    self.s_in.wait_event(buf_free[b])       # the compute that last used these buffers is done
                dev = [buf[:, :n] for buf in stage[b]]
                for d, h in zip(dev, ins):
                    d.copy_(h[:, lo:hi], non_blocking=True)
                in_ready[b].record(self.s_in)
            compute.wait_event(in_ready[b])
            qd, kd, vd = dev[:3]
            if rope is not None:      # rotated copies handed from forward to backward
                o, lse, q_rot, k_rot = swa_forward_rot(qd, kd, vd, rope, *window, sm_scale)
                res = (o,)
                if with_bwd:
                    res += tuple(swa_backward_rot(q_rot, k_rot, vd, o, lse, dev[3], rope, *window, sm_scale))
            else:
                o, lse = swa_forward(qd, kd, vd, None, *window, sm_scale)
                res = (o,)
                if with_bwd:
                    res += tuple(swa_backward(qd, kd, vd, o, lse, dev[3], None, *window, sm_scale))
            ev = torch.cuda.Event()
            ev.record(compute)
            buf_free[b] = ev
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev)
                for r, h in zip(res, outs):
                    if h is not None:
                        h[:, lo:hi].copy_(r, non_blocking=True)
                        r.record_stream(self.s_out)
                oe = torch.cuda.Event()
                oe.record(self.s_out)
                out_events.append(oe)
        # ``done`` = the last copy-out, which follows every kernel and every copy-in of this run.  The compute stream
        # itself is NOT made to wait for the copy-out: that would drain the pipeline between consecutive runs (the
        # next run's first kernels, and with them its copies, would start only after this run's last bytes had
        # reached the host -- about one chunk's copy time per run).
        self.done.record(self.s_out)
        return outs
