"""Fastmax attention for callers whose tensors live in HOST memory.

The reference's callers hand the operator whatever the surrounding script holds and move it to the GPU right
before the call (`token_chunk.to("cuda")`, transformer/eval.py:14-16).  When q, k, v and the upstream gradient
sit in (pinned) host memory, a forward+backward of BASELINE-sized tensors spends more time on PCIe than on
the GPU: 268 MB in, 268 MB out, 3 ms of kernels.  `HostFastmax` therefore cuts the batch into pieces and runs
three stages on three streams: piece i+1 is copied in while piece i computes and piece i-1 is copied out.
Every (batch, head) is independent, so the results are those of one call over the whole batch.
"""
from __future__ import annotations

import math

import torch

from . import _lib


class HostFastmax:
    """forward_backward(hq, hk, hv, hdo, ho, hdq, hdk, hdv): all arguments (b, h, n, d) HOST tensors (pinned memory
    for asynchronous copies); the last four receive the output and the three gradients.

    mask, temperature, a0, a1, a2, p: as in `fastmax_custom`.  pieces: how many batch slices to pipeline (default:
    one per batch entry, at most 8).  Device buffers for the whole batch are kept between calls.
    """

    def __init__(self, mask=True, temperature=1.0, a0=1.0, a1=1.0, a2=0.5, p=2, pieces=None, device=None):
        self.mask = bool(mask)
        self.inv_temperature = 1.0 / float(temperature)
        self.a0, self.a1, self.a2, self.p = float(a0), float(a1), float(a2), int(p)
        self.pieces = pieces
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._s_in = torch.cuda.Stream(self.device)
        self._s_out = torch.cuda.Stream(self.device)
        self._bufs = None

    def _device_buffers(self, ref):
        key = (tuple(ref.shape), ref.dtype)
        if self._bufs is None or self._bufs[0] != key:
            self._bufs = (key, [torch.empty(ref.shape, dtype=ref.dtype, device=self.device) for _ in range(4)])
        return self._bufs[1]

    def forward_backward(self, hq, hk, hv, hdo, ho, hdq, hdk, hdv):
        for t in (hq, hk, hv, hdo, ho, hdq, hdk, hdv):
            if t.is_cuda or t.dim() != 4:
                raise ValueError("HostFastmax takes (b, h, n, d) host tensors")
        if hk.shape != hv.shape or hq.shape != hdo.shape:
            raise ValueError("k/v and q/d_out shapes must agree")
        B = hq.shape[0]
        npieces = min(B, 8) if self.pieces is None else max(1, min(int(self.pieces), B))
        per = math.ceil(B / npieces)
        same = hq.shape == hk.shape
        dq_, dk_, dv_, ddo = self._device_buffers(hq) if same else (
            torch.empty(hq.shape, dtype=hq.dtype, device=self.device), torch.empty(hk.shape, dtype=hk.dtype, device=self.device),
            torch.empty(hv.shape, dtype=hv.dtype, device=self.device), torch.empty(hdo.shape, dtype=hdo.dtype, device=self.device))
        cur = torch.cuda.current_stream(self.device)
        # whatever the caller queued on its stream (earlier use of the host buffers) is ordered before the copies
        start = torch.cuda.Event()
        start.record(cur)
        self._s_in.wait_event(start)
        self._s_out.wait_event(start)
        keep = []   # results stay referenced until the copies that read them have finished
        for b0 in range(0, B, per):
            sl = slice(b0, min(B, b0 + per))
            with torch.cuda.stream(self._s_in):
                for dst, src in ((dq_, hq), (dk_, hk), (dv_, hv), (ddo, hdo)):
                    dst[sl].copy_(src[sl], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self._s_in)
            cur.wait_event(ready)
            o, g, _ = _lib.forward(dq_[sl], dk_[sl], dv_[sl], self.mask, self.inv_temperature, self.a0, self.a1, self.a2, self.p)
            gq, gk, gv, _ = _lib.backward(dq_[sl], dk_[sl], dv_[sl], o, g, ddo[sl], self.mask, self.inv_temperature, self.a0,
                                          self.a1, self.a2, self.p)
            done = torch.cuda.Event()
            done.record(cur)
            keep.append((o, g, gq, gk, gv))
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(done)
                for dst, src in ((ho, o), (hdq, gq), (hdk, gk), (hdv, gv)):
                    dst[sl].copy_(src, non_blocking=True)
        fin = torch.cuda.Event()
        fin.record(self._s_out)
        cur.wait_event(fin)         # the caller's stream sees the host results once it passes this point
        self._s_in.wait_event(fin)  # the next call's copies must not overwrite device inputs still in use
        cur.synchronize()
        del keep
        return ho, hdq, hdk, hdv
