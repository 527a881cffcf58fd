"""Forward + backward of the Field read for data that lives in host memory.

``HostFieldRead`` streams a batch from pinned host tensors through the GPU and back in
row chunks on three CUDA streams, so the upload of chunk i+1, the kernels of chunk i and
the download of chunk i-1 overlap and both PCIe directions stay busy. Dependencies are
tracked per tensor, not per chunk: the forward starts when ``raw`` has landed, ``read``
leaves while ``grad_read`` is still arriving, ``grad_raw`` follows the backward; with
``wait=False`` consecutive calls overlap as well. Results are the same as one call of the
operator on the whole batch: the recurrence never mixes batch rows, and the parameter
gradients are sums over rows, accumulated chunk by chunk in a fixed order.
"""
from __future__ import annotations

import torch

from . import _lib


class HostFieldRead:
    def __init__(self, device, batch: int, length: int, channels: int, rows_per_chunk: int = 1,
                 slots: int = 2):
        self.lib = _lib.load()
        self.device = torch.device(device)
        self.B, self.L, self.C = batch, length, channels
        self.rows = max(1, min(rows_per_chunk, batch))
        r, L, C = self.rows, length, channels
        f32 = dict(device=self.device, dtype=torch.float32)
        self.slots = []
        for _ in range(max(2, slots)):
            self.slots.append(dict(
                raw=torch.empty(r, L, 3 * C, **f32), grad=torch.empty(r, L, 4 * C, **f32),
                read=torch.empty(r, L, 4 * C, **f32), graw=torch.empty(r, L, 3 * C, **f32),
                gpar=torch.empty(3, C, **f32),
                raw_loaded=torch.cuda.Event(), loaded=torch.cuda.Event(),
                forward_done=torch.cuda.Event(), computed=torch.cuda.Event(),
                stored=torch.cuda.Event()))
        self.nf = self.lib.fields_read_workspace_bytes(r, L, C, 0)
        self.nb = self.lib.fields_read_workspace_bytes(r, L, C, 1)
        self.ws = torch.empty(max(self.nf, self.nb, 256), dtype=torch.uint8, device=self.device)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        # two accumulators for the parameter gradients, used by alternate calls, so that a call may
        # start while the previous call's result is still on its way to the host
        self.gpar = [torch.zeros(3, C, **f32) for _ in range(2)]
        self.gpar_free = [torch.cuda.Event() for _ in range(2)]
        self.calls = 0

    def fwd_bwd(self, raw_host, grad_host, tr, ti, gamma, read_host, graw_host, gpar_host=None,
                wait: bool = True) -> torch.Tensor:
        """All host tensors pinned: raw [B,L,3C], grad_read [B,L,4C] in; read, grad_raw out.
        Returns the parameter gradients ``[3, C]`` (d lambda_r, d lambda_i, d gamma) on the device
        and, if ``gpar_host`` (pinned ``[3, C]``) is given, also copies them there.

        With ``wait`` the caller's current stream waits for everything before control returns to
        it. With ``wait=False`` it does not: the next call may then start uploading while this
        call's results are still being downloaded (the two PCIe directions overlap across calls
        too); call :meth:`join` before touching the host outputs, and pass ``gpar_host`` - the
        returned device tensor is reused by the call after next."""
        lib, L, C = self.lib, self.L, self.C
        main = torch.cuda.current_stream(self.device)
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_stream(main)
        which = self.calls % 2
        self.calls += 1
        gpar_total = self.gpar[which]
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.gpar_free[which])   # its last result has left
            gpar_total.zero_()
        trp, tip, gmp = tr.data_ptr(), ti.data_ptr(), gamma.data_ptr()
        for i, lo in enumerate(range(0, self.B, self.rows)):
            hi = min(lo + self.rows, self.B)
            n = hi - lo
            s = self.slots[i % len(self.slots)]
            # Finer than one event per chunk: the forward needs only `raw`, and `read` can leave as
            # soon as the forward is done, while `grad_read` is still arriving; `grad_raw` follows
            # the backward. That shortens the phases in which only one copy direction is busy.
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(s["computed"])      # kernels of the slot's last use are done
                s["raw"][:n].copy_(raw_host[lo:hi], non_blocking=True)
                s["raw_loaded"].record(self.s_in)
                s["grad"][:n].copy_(grad_host[lo:hi], non_blocking=True)
                s["loaded"].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(s["raw_loaded"])
                self.s_run.wait_event(s["stored"])       # the slot's last results have left
                q = self.s_run.cuda_stream
                rc = lib.fields_read_forward(s["raw"].data_ptr(), trp, tip, gmp, None,
                                             s["read"].data_ptr(), None, self.ws.data_ptr(),
                                             self.nf, n, L, C, q)
                _lib.check(rc, "fields_read_forward")
                s["forward_done"].record(self.s_run)
                self.s_run.wait_event(s["loaded"])
                g = s["gpar"]
                rc = lib.fields_read_backward(s["raw"].data_ptr(), trp, tip, gmp, None,
                                              s["read"].data_ptr(), s["grad"].data_ptr(), None,
                                              s["graw"].data_ptr(), g[0].data_ptr(), g[1].data_ptr(),
                                              g[2].data_ptr(), None, self.ws.data_ptr(), self.nb,
                                              n, L, C, q)
                _lib.check(rc, "fields_read_backward")
                gpar_total.add_(g)
                s["computed"].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(s["forward_done"])
                read_host[lo:hi].copy_(s["read"][:n], non_blocking=True)
                self.s_out.wait_event(s["computed"])
                graw_host[lo:hi].copy_(s["graw"][:n], non_blocking=True)
                s["stored"].record(self.s_out)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_run)
            if gpar_host is not None:
                gpar_host.copy_(gpar_total, non_blocking=True)
            self.gpar_free[which].record(self.s_out)
        if wait:
            self.join()
        return gpar_total

    def join(self):
        """Makes the caller's current stream wait for every call issued so far."""
        main = torch.cuda.current_stream(self.device)
        for st in (self.s_in, self.s_run, self.s_out):
            main.wait_stream(st)
