"""Sequence-sharded Field read (forward, and backward for training) across the GPUs of one node.

A long sequence is cut into P contiguous spans, one per rank. The recurrence is an
affine map per (batch, channel), so a span is summarised by one complex pair
``s_out = A s_in + Bv``: ranks exchange those pairs (``[B, 4, C]`` floats each, 8 KB at
B = 1), every rank folds the pairs of the spans before it onto the initial state and
then runs its span from that state. Everything else in a Field block is token-parallel.
The reference runs a sequence on one GPU only; its single-device full-sequence output is
the oracle for this path.

Steps on rank r (all on the current CUDA stream):
  1. ``fields_read_span_summary``  - one read of the span, chunk maps composed to (A, Bv);
  2. ``all_gather`` of the summaries over NCCL (NVLink/NVSwitch);
  3. ``fields_read_fold_summaries`` - state entering span r;
  4. ``fields_read_forward`` with that state.

The backward pass mirrors this in reverse rank order (``sequence_parallel_field_read_autograd``):
the gradient carry is an affine map per span as well (``carry_in = P carry_out + Q``), so ranks
exchange dual summaries, every rank folds the spans AFTER it, last first, and runs
``fields_read_backward`` on its span with that carry; the three parameter gradients are sums
over spans (one all-reduce of 3 C floats).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


class CudaOps:
    """The three device operations, on the CUDA library."""

    def span_summary(self, raw, tr, ti, gamma):
        lib = _lib.load()
        B, L, C3 = raw.shape
        C = C3 // 3
        out = torch.empty((B, 4, C), device=raw.device, dtype=torch.float32)
        n = lib.fields_read_workspace_bytes(B, L, C, 0)
        ws = torch.empty(max(n, 256), dtype=torch.uint8, device=raw.device)
        rc = lib.fields_read_span_summary(raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                          gamma.data_ptr(), out.data_ptr(), ws.data_ptr(), n,
                                          B, L, C, torch.cuda.current_stream(raw.device).cuda_stream)
        _lib.check(rc, "fields_read_span_summary")
        return out

    def fold(self, summaries, rank, state0):
        lib = _lib.load()
        P, B, _, C = summaries.shape
        out = torch.empty((B, 2 * C), device=summaries.device, dtype=torch.float32)
        rc = lib.fields_read_fold_summaries(
            summaries.data_ptr(), None if state0 is None else state0.data_ptr(), out.data_ptr(),
            rank, P, B, C, torch.cuda.current_stream(summaries.device).cuda_stream)
        _lib.check(rc, "fields_read_fold_summaries")
        return out

    def forward(self, raw, tr, ti, gamma, state_in):
        from .field_read import field_read_with_state
        with torch.no_grad():
            return field_read_with_state(raw, tr, ti, gamma, state_in)

    def span_summary_backward(self, raw, tr, ti, grad_read):
        lib = _lib.load()
        B, L, C3 = raw.shape
        C = C3 // 3
        out = torch.empty((B, 4, C), device=raw.device, dtype=torch.float32)
        n = lib.fields_read_workspace_bytes(B, L, C, 1)
        ws = torch.empty(max(n, 256), dtype=torch.uint8, device=raw.device)
        rc = lib.fields_read_span_summary_backward(
            raw.data_ptr(), tr.data_ptr(), ti.data_ptr(), grad_read.data_ptr(), out.data_ptr(),
            ws.data_ptr(), n, B, L, C, torch.cuda.current_stream(raw.device).cuda_stream)
        _lib.check(rc, "fields_read_span_summary_backward")
        return out

    def fold_backward(self, summaries, rank, carry_end):
        lib = _lib.load()
        P, B, _, C = summaries.shape
        out = torch.empty((B, 2 * C), device=summaries.device, dtype=torch.float32)
        rc = lib.fields_read_fold_summaries_backward(
            summaries.data_ptr(), None if carry_end is None else carry_end.data_ptr(),
            out.data_ptr(), rank, P, B, C,
            torch.cuda.current_stream(summaries.device).cuda_stream)
        _lib.check(rc, "fields_read_fold_summaries_backward")
        return out

    def backward(self, raw, tr, ti, gamma, read, grad_read, state_in, grad_state_out):
        """Returns ``(grad_raw, grad_params [3, C], grad_state_in [B, 2C])`` of one span."""
        lib = _lib.load()
        B, L, C3 = raw.shape
        C = C3 // 3
        grad_raw = torch.empty_like(raw)
        g_par = torch.empty((3, C), device=raw.device, dtype=torch.float32)
        g_sin = torch.empty((B, 2 * C), device=raw.device, dtype=torch.float32)
        n = lib.fields_read_workspace_bytes(B, L, C, 1)
        ws = torch.empty(max(n, 256), dtype=torch.uint8, device=raw.device)
        rc = lib.fields_read_backward(
            raw.data_ptr(), tr.data_ptr(), ti.data_ptr(), gamma.data_ptr(),
            None if state_in is None else state_in.data_ptr(), read.data_ptr(),
            grad_read.data_ptr(), None if grad_state_out is None else grad_state_out.data_ptr(),
            grad_raw.data_ptr(), g_par[0].data_ptr(), g_par[1].data_ptr(), g_par[2].data_ptr(),
            g_sin.data_ptr(), ws.data_ptr(), n, B, L, C,
            torch.cuda.current_stream(raw.device).cuda_stream)
        _lib.check(rc, "fields_read_backward")
        return grad_raw, g_par, g_sin


class SequenceParallelForward:
    """The same four steps on preallocated buffers, for repeated calls on one span shape.

    Holds the outputs (``read``, ``state_out``), the summary buffers and the workspace, so a
    call costs three C-ABI launches and one NCCL all_gather and allocates nothing.
    """

    def __init__(self, batch: int, span_length: int, channels: int, device, group=None):
        self.lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.B, self.L, self.C = batch, span_length, channels
        f32 = dict(device=device, dtype=torch.float32)
        self.summary = torch.empty(batch, 4, channels, **f32)
        self.gathered = torch.empty(self.world * batch, 4, channels, **f32)
        self.state_in = torch.empty(batch, 2 * channels, **f32)
        self.state_out = torch.empty(batch, 2 * channels, **f32)
        self.read = torch.empty(batch, span_length, 4 * channels, **f32)
        self.nbytes = self.lib.fields_read_workspace_bytes(batch, span_length, channels, 0)
        self.ws = torch.empty(max(self.nbytes, 256), dtype=torch.uint8, device=device)
        self.device = torch.device(device)

    def __call__(self, raw_span, tr, ti, gamma, state0: Optional[torch.Tensor] = None):
        lib, B, L, C = self.lib, self.B, self.L, self.C
        if tuple(raw_span.shape) != (B, L, 3 * C) or not raw_span.is_contiguous():
            raise ValueError(f"expected a contiguous [{B}, {L}, {3 * C}] span")
        st = torch.cuda.current_stream(self.device).cuda_stream
        args = (raw_span.data_ptr(), tr.data_ptr(), ti.data_ptr(), gamma.data_ptr())
        state_in = None if state0 is None else state0.data_ptr()
        if self.world > 1:
            rc = lib.fields_read_span_summary(*args, self.summary.data_ptr(), self.ws.data_ptr(),
                                              self.nbytes, B, L, C, st)
            _lib.check(rc, "fields_read_span_summary")
            dist.all_gather_into_tensor(self.gathered, self.summary, group=self.group)
            rc = lib.fields_read_fold_summaries(self.gathered.data_ptr(), state_in,
                                                self.state_in.data_ptr(), self.rank, self.world,
                                                B, C, st)
            _lib.check(rc, "fields_read_fold_summaries")
            state_in = self.state_in.data_ptr()
        rc = lib.fields_read_forward(*args, state_in, self.read.data_ptr(),
                                     self.state_out.data_ptr(), self.ws.data_ptr(), self.nbytes,
                                     B, L, C, st)
        _lib.check(rc, "fields_read_forward")
        return self.read, self.state_out


class SequenceParallelTrainStep:
    """Forward and backward of one rank's span on preallocated buffers (NCCL exchanges).

    ``forward`` is :class:`SequenceParallelForward`; ``backward`` mirrors it in reverse rank
    order: dual span summary, all_gather, reverse fold, ``fields_read_backward`` with the folded
    carry, all_reduce of the three parameter gradients. Seven C-ABI launches and three NCCL calls
    per step, no allocation.
    """

    def __init__(self, batch: int, span_length: int, channels: int, device, group=None):
        self.fwd = SequenceParallelForward(batch, span_length, channels, device, group)
        f = self.fwd
        f32 = dict(device=device, dtype=torch.float32)
        self.dual = torch.empty(batch, 4, channels, **f32)
        self.gathered_dual = torch.empty(f.world * batch, 4, channels, **f32)
        self.carry = torch.empty(batch, 2 * channels, **f32)
        self.grad_raw = torch.empty(batch, span_length, 3 * channels, **f32)
        self.grad_par = torch.empty(3, channels, **f32)
        self.nbytes_bwd = f.lib.fields_read_workspace_bytes(batch, span_length, channels, 1)
        self.ws_bwd = torch.empty(max(self.nbytes_bwd, 256), dtype=torch.uint8, device=device)
        self.had_state0 = False

    def forward(self, raw_span, tr, ti, gamma, state0: Optional[torch.Tensor] = None):
        self.had_state0 = state0 is not None
        self.state0 = state0
        return self.fwd(raw_span, tr, ti, gamma, state0)

    def backward(self, raw_span, tr, ti, gamma, grad_read_span):
        """Gradients of the last ``forward``: ``(grad_raw_span, grad_params [3, C])``; the
        parameter gradients are summed over the ranks."""
        f = self.fwd
        lib, B, L, C = f.lib, f.B, f.L, f.C
        if tuple(grad_read_span.shape) != (B, L, 4 * C) or not grad_read_span.is_contiguous():
            raise ValueError(f"expected a contiguous [{B}, {L}, {4 * C}] gradient")
        st = torch.cuda.current_stream(f.device).cuda_stream
        args = (raw_span.data_ptr(), tr.data_ptr(), ti.data_ptr())
        carry = None
        if f.world > 1:
            rc = lib.fields_read_span_summary_backward(*args, grad_read_span.data_ptr(),
                                                       self.dual.data_ptr(), self.ws_bwd.data_ptr(),
                                                       self.nbytes_bwd, B, L, C, st)
            _lib.check(rc, "fields_read_span_summary_backward")
            dist.all_gather_into_tensor(self.gathered_dual, self.dual, group=f.group)
            rc = lib.fields_read_fold_summaries_backward(self.gathered_dual.data_ptr(), None,
                                                         self.carry.data_ptr(), f.rank, f.world,
                                                         B, C, st)
            _lib.check(rc, "fields_read_fold_summaries_backward")
            carry = self.carry.data_ptr()
            state_in = f.state_in.data_ptr()
        else:
            state_in = self.state0.data_ptr() if self.had_state0 else None
        g = self.grad_par
        rc = lib.fields_read_backward(*args, gamma.data_ptr(), state_in, f.read.data_ptr(),
                                      grad_read_span.data_ptr(), carry, self.grad_raw.data_ptr(),
                                      g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), None,
                                      self.ws_bwd.data_ptr(), self.nbytes_bwd, B, L, C, st)
        _lib.check(rc, "fields_read_backward")
        if f.world > 1:
            dist.all_reduce(g, group=f.group)
        return self.grad_raw, g


class SequenceParallelForwardP2P:
    """Sequence-sharded forward whose summary exchange goes through peer memory, not NCCL.

    Each rank owns a mailbox in symmetric memory (``torch.distributed._symmetric_memory``:
    every GPU of the node can write it over NVLink). ``fields_read_span_summary_put`` stores the
    rank's span summary, tagged with a per-call epoch, straight into every rank's mailbox;
    ``fields_read_fold_mailbox`` waits (bounded) for all summaries of that epoch and folds the
    earlier ranks onto the initial state; ``fields_read_forward`` runs the span from there.
    Three launches of this library per call, no collective, nothing to clear between calls.
    A summary that never arrives turns into a NaN state and a non-zero status word
    (:meth:`status`), never into a hang. The calls carry the epoch as a kernel argument, so
    they must not be replayed from a captured CUDA graph.
    """

    def __init__(self, batch: int, span_length: int, channels: int, device, group=None,
                 max_polls: int = 0):
        import ctypes
        import os
        self.max_polls = int(max_polls)  # bound of the device-side waits; 0: about a second
        # The mailboxes are written with plain peer stores only; binding them to an NVLink
        # multicast object buys nothing and ties every rank's memory to the others' lifetime.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.lib = _lib.load()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.B, self.L, self.C = batch, span_length, channels
        self.device = torch.device(device)
        f32 = dict(device=self.device, dtype=torch.float32)
        nbytes = self.lib.fields_read_mailbox_bytes(self.world, batch, channels)
        self.mail = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=self.device)
        self.mail.zero_()
        self.handle = symm_mem.rendezvous(self.mail, self.group)
        self.peers = (ctypes.c_void_p * self.world)(*[int(a) for a in self.handle.buffer_ptrs])
        self.error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.state_in = torch.empty(batch, 2 * channels, **f32)
        self.state_out = torch.empty(batch, 2 * channels, **f32)
        self.read = torch.empty(batch, span_length, 4 * channels, **f32)
        self.nbytes = self.lib.fields_read_workspace_bytes(batch, span_length, channels, 0)
        self.ws = torch.empty(max(self.nbytes, 256), dtype=torch.uint8, device=self.device)
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every mailbox is zeroed before anyone writes into it

    def __call__(self, raw_span, tr, ti, gamma, state0: Optional[torch.Tensor] = None):
        lib, B, L, C = self.lib, self.B, self.L, self.C
        if tuple(raw_span.shape) != (B, L, 3 * C) or not raw_span.is_contiguous():
            raise ValueError(f"expected a contiguous [{B}, {L}, {3 * C}] span")
        self.epoch = self.epoch + 1 if self.epoch < 0xFFFFFFFE else 1
        st = torch.cuda.current_stream(self.device).cuda_stream
        args = (raw_span.data_ptr(), tr.data_ptr(), ti.data_ptr(), gamma.data_ptr())
        rc = lib.fields_read_span_summary_put(*args, self.peers, None, self.rank, self.world,
                                              self.epoch, self.ws.data_ptr(), self.nbytes, B, L, C, st)
        _lib.check(rc, "fields_read_span_summary_put")
        rc = lib.fields_read_fold_mailbox(self.mail.data_ptr(),
                                          None if state0 is None else state0.data_ptr(),
                                          self.state_in.data_ptr(), self.error.data_ptr(),
                                          self.rank, self.world, self.epoch, self.max_polls, B, C, st)
        _lib.check(rc, "fields_read_fold_mailbox")
        rc = lib.fields_read_forward(*args, self.state_in.data_ptr(), self.read.data_ptr(),
                                     self.state_out.data_ptr(), self.ws.data_ptr(), self.nbytes,
                                     B, L, C, st)
        _lib.check(rc, "fields_read_forward")
        return self.read, self.state_out

    def status(self) -> int:
        """0, or 1 if some call since construction gave up waiting for a peer's summary (syncs)."""
        return int(self.error.item())

    def check_status(self) -> None:
        """Raises if a device-side wait of this object ever ran out (one small device-to-host
        read: call it where the step synchronises anyway, e.g. next to reading the loss).

        The waits tolerate about a second of skew between the ranks by default (``max_polls``
        of the constructor, in polls of well under a microsecond each). A rank that is later
        than that - a checkpoint write, a stalled loader - makes the others give up: their
        outputs hold NaN from that call on, never stale data, and this method reports it."""
        if self.status():
            raise _lib.FieldsLibraryError(
                "a sequence-parallel exchange gave up waiting for a peer's summary "
                f"(FIELDS_ERR_TIMEOUT, rank {self.rank} of {self.world}): outputs since then hold NaN")


class SequenceParallelForwardFused(SequenceParallelForwardP2P):
    """Sequence-sharded forward in ONE launch per rank (``fields_read_forward_sharded``).

    Same mailboxes, epochs and results as :class:`SequenceParallelForwardP2P`, but the span's
    summary sweep, the exchange over NVLink peer stores, the fold and the forward pass are one
    cooperative kernel: the span is read from HBM once when its ``raw`` fits the L2 cache (the
    second sweep starts with the rows the first one read last), and there are no launch gaps
    between the stages. ``max_polls`` bounds every device-side wait (0: the library's default,
    about a second of rank skew); a wait that runs out sets the status word and leaves NaN in
    the outputs instead of hanging. By default the epoch is a kernel argument, so the call must
    not be replayed from a captured CUDA graph; with ``device_epoch=True`` the epoch lives in the
    rank's mailbox and the kernel advances it itself: the call can then be captured and
    replayed (every rank replays the same number of times), and this object's mailboxes must
    not be used by calls that pass their own epochs.
    """

    def __init__(self, batch: int, span_length: int, channels: int, device, group=None,
                 max_polls: int = 0, device_epoch: bool = False):
        super().__init__(batch, span_length, channels, device, group, max_polls)
        self.device_epoch = bool(device_epoch)

    def __call__(self, raw_span, tr, ti, gamma, state0: Optional[torch.Tensor] = None):
        B, L, C = self.B, self.L, self.C
        if tuple(raw_span.shape) != (B, L, 3 * C) or not raw_span.is_contiguous():
            raise ValueError(f"expected a contiguous [{B}, {L}, {3 * C}] span")
        if not self.device_epoch:
            self.epoch = self.epoch + 1 if self.epoch < 0xFFFFFFFE else 1
        rc = self.lib.fields_read_forward_sharded(
            raw_span.data_ptr(), tr.data_ptr(), ti.data_ptr(), gamma.data_ptr(),
            None if state0 is None else state0.data_ptr(), self.read.data_ptr(),
            self.state_out.data_ptr(), None, self.peers, self.error.data_ptr(), self.rank,
            self.world, 0 if self.device_epoch else self.epoch, self.max_polls, B, L, C,
            torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "fields_read_forward_sharded")
        return self.read, self.state_out


class SequenceParallelTrainStepP2P(SequenceParallelForwardP2P):
    """Forward and backward of one rank's span with both exchanges through peer memory.

    Calling the object runs the forward (as :class:`SequenceParallelForwardP2P`); ``backward``
    puts the span's dual summary into every mailbox under the next epoch
    (``fields_read_span_summary_backward_put``), waits with a bound for all of them and folds
    the later spans, last first (``fields_read_fold_mailbox_backward``), and runs
    ``fields_read_backward`` with that carry. The 3 C parameter-gradient sums (and the ranks'
    status words beside them) are added over the ranks through the same mailboxes too
    (``fields_read_sum_over_ranks``: peer stores, bounded wait, addition in rank order, so every
    rank holds the same bits); ``nccl_reduce=True`` sends them through one NCCL all_reduce
    instead. Like the forward, not for replay from a captured CUDA graph.
    """

    def __init__(self, batch: int, span_length: int, channels: int, device, group=None,
                 max_polls: int = 0, nccl_reduce: bool = False):
        super().__init__(batch, span_length, channels, device, group, max_polls)
        self.nccl_reduce = bool(nccl_reduce)
        f32 = dict(device=self.device, dtype=torch.float32)
        self.carry = torch.empty(batch, 2 * channels, **f32)
        self.addends = torch.zeros(3 * channels + 1, **f32)
        self.grad_raw = torch.empty(batch, span_length, 3 * channels, **f32)
        # [3 C] parameter gradients + one word: the ranks' error words, summed by the same
        # all_reduce, so every rank learns of a timeout anywhere without another collective
        self.reduced = torch.zeros(3 * channels + 1, **f32)
        self.grad_par = self.reduced[:3 * channels].view(3, channels)
        self.nbytes_bwd = self.lib.fields_read_workspace_bytes(batch, span_length, channels, 1)
        self.ws_bwd = torch.empty(max(self.nbytes_bwd, 256), dtype=torch.uint8, device=self.device)

    def forward(self, raw_span, tr, ti, gamma, state0: Optional[torch.Tensor] = None):
        return self(raw_span, tr, ti, gamma, state0)

    def backward(self, raw_span, tr, ti, gamma, grad_read_span):
        """Gradients of the last forward: ``(grad_raw_span, grad_params [3, C])``, the parameter
        gradients summed over the ranks."""
        lib, B, L, C = self.lib, self.B, self.L, self.C
        if tuple(grad_read_span.shape) != (B, L, 4 * C) or not grad_read_span.is_contiguous():
            raise ValueError(f"expected a contiguous [{B}, {L}, {4 * C}] gradient")
        self.epoch = self.epoch + 1 if self.epoch < 0xFFFFFFFE else 1
        st = torch.cuda.current_stream(self.device).cuda_stream
        args = (raw_span.data_ptr(), tr.data_ptr(), ti.data_ptr())
        rc = lib.fields_read_span_summary_backward_put(*args, grad_read_span.data_ptr(), self.peers,
                                                       None, self.rank, self.world, self.epoch,
                                                       self.ws_bwd.data_ptr(), self.nbytes_bwd,
                                                       B, L, C, st)
        _lib.check(rc, "fields_read_span_summary_backward_put")
        rc = lib.fields_read_fold_mailbox_backward(self.mail.data_ptr(), None, self.carry.data_ptr(),
                                                   self.error.data_ptr(), self.rank, self.world,
                                                   self.epoch, self.max_polls, B, C, st)
        _lib.check(rc, "fields_read_fold_mailbox_backward")
        g = self.grad_par
        # this rank's sums land in `addends` when they still have to cross the ranks
        own = self.addends[:3 * C].view(3, C) if self.world > 1 and not self.nccl_reduce else g
        rc = lib.fields_read_backward(*args, gamma.data_ptr(), self.state_in.data_ptr(),
                                      self.read.data_ptr(), grad_read_span.data_ptr(),
                                      self.carry.data_ptr(), self.grad_raw.data_ptr(),
                                      own[0].data_ptr(), own[1].data_ptr(), own[2].data_ptr(), None,
                                      self.ws_bwd.data_ptr(), self.nbytes_bwd, B, L, C, st)
        _lib.check(rc, "fields_read_backward")
        if self.world > 1 and self.nccl_reduce:
            self.reduced[-1:].copy_(self.error)
            dist.all_reduce(self.reduced, group=self.group)
        elif self.world > 1:
            self.addends[-1:].copy_(self.error)
            self.epoch = self.epoch + 1 if self.epoch < 0xFFFFFFFE else 1
            rc = lib.fields_read_sum_over_ranks(self.addends.data_ptr(), self.reduced.data_ptr(),
                                                3 * C + 1, self.peers, self.error.data_ptr(),
                                                self.rank, self.world, self.epoch, self.max_polls,
                                                B, C, st)
            _lib.check(rc, "fields_read_sum_over_ranks")
        return self.grad_raw, g

    def status(self) -> int:
        """Number of ranks whose waits have run out, as of the last backward (syncs); before the
        first backward, this rank's own error word."""
        seen = float(self.reduced[-1].item())
        if seen != seen:          # the sum itself gave up waiting: NaN
            return self.world
        return int(seen) or int(self.error.item())


def span_bounds(length: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, near-equal spans: the first ``length % world`` ranks get one step more."""
    base, extra = divmod(length, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sequence_parallel_field_read(raw_span: torch.Tensor, tr: torch.Tensor, ti: torch.Tensor,
                                 gamma: torch.Tensor, group=None,
                                 state0: Optional[torch.Tensor] = None, ops=None):
    """Forward of this rank's span of a sequence sharded over ``group``.

    ``raw_span`` is ``[B, L_r, 3C]`` fp32 (spans may differ in length but not be empty);
    ``state0`` is the state before the first span (same on every rank, or None for zero).
    Returns ``(read_span [B, L_r, 4C], state_after_span [B, 2C])``.
    """
    ops = ops or CudaOps()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if raw_span.dim() != 3 or raw_span.shape[1] == 0:
        raise ValueError(f"every rank needs a non-empty span, got {tuple(raw_span.shape)}")
    raw_span = raw_span.contiguous()
    if world == 1:
        return ops.forward(raw_span, tr, ti, gamma, state0)
    summary = ops.span_summary(raw_span, tr, ti, gamma)
    B = summary.shape[0]
    gathered = torch.empty((world * B,) + tuple(summary.shape[1:]), device=summary.device,
                           dtype=summary.dtype)
    dist.all_gather_into_tensor(gathered, summary, group=group)  # rank-major along dim 0
    state_in = ops.fold(gathered.view(world, B, *summary.shape[1:]), rank, state0)
    return ops.forward(raw_span, tr, ti, gamma, state_in)


def _gather_summaries(summary: torch.Tensor, world: int, group) -> torch.Tensor:
    B = summary.shape[0]
    gathered = torch.empty((world * B,) + tuple(summary.shape[1:]), device=summary.device,
                           dtype=summary.dtype)
    dist.all_gather_into_tensor(gathered, summary.contiguous(), group=group)  # rank-major
    return gathered.view(world, B, *summary.shape[1:])


class _SequenceParallelFieldRead(torch.autograd.Function):
    """read_span = F(raw_span, tr, ti, gamma) for one rank's span, differentiable across ranks."""

    @staticmethod
    def forward(ctx, raw_span, tr, ti, gamma, state0, group, ops, reduce_parameter_grads):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        raw_span = raw_span.contiguous().float()
        tr, ti, gamma = (t.contiguous().float() for t in (tr, ti, gamma))
        state_in = state0
        if world > 1:
            gathered = _gather_summaries(ops.span_summary(raw_span, tr, ti, gamma), world, group)
            state_in = ops.fold(gathered, rank, state0)
        read, _ = ops.forward(raw_span, tr, ti, gamma, state_in)
        ctx.save_for_backward(raw_span, tr, ti, gamma, read,
                              state_in if state_in is not None else torch.empty(0))
        ctx.group, ctx.ops, ctx.reduce = group, ops, reduce_parameter_grads
        return read

    @staticmethod
    def backward(ctx, grad_read):
        raw_span, tr, ti, gamma, read, state_in = ctx.saved_tensors
        state_in = state_in if state_in.numel() else None
        group, ops = ctx.group, ctx.ops
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        grad_read = grad_read.contiguous().float()
        carry = None
        if world > 1:
            dual = ops.span_summary_backward(raw_span, tr, ti, grad_read)
            carry = ops.fold_backward(_gather_summaries(dual, world, group), rank, None)
        grad_raw, g_par, _ = ops.backward(raw_span, tr, ti, gamma, read, grad_read, state_in, carry)
        if world > 1 and ctx.reduce:
            dist.all_reduce(g_par, group=group)
        return grad_raw, g_par[0], g_par[1], g_par[2], None, None, None, None


def sequence_parallel_field_read_autograd(raw_span: torch.Tensor, tr: torch.Tensor,
                                          ti: torch.Tensor, gamma: torch.Tensor, group=None,
                                          state0: Optional[torch.Tensor] = None, ops=None,
                                          reduce_parameter_grads: bool = True) -> torch.Tensor:
    """Differentiable forward of this rank's span of a sequence sharded over ``group``.

    ``loss.backward()`` on every rank exchanges the dual span summaries (one all_gather of
    ``[B, 4, C]`` per rank), so ``raw_span.grad`` equals the corresponding slice of the
    single-device gradient. The gradients of ``tr``, ``ti`` and ``gamma`` are sums over the
    spans: with ``reduce_parameter_grads`` they are all-reduced here and every rank gets the
    full gradient; without it each rank keeps its span's share (for callers whose data-parallel
    wrapper already sums replicated parameters over this group). ``state0`` (the state before
    the first span) is treated as a constant.
    """
    if raw_span.dim() != 3 or raw_span.shape[1] == 0:
        raise ValueError(f"every rank needs a non-empty span, got {tuple(raw_span.shape)}")
    return _SequenceParallelFieldRead.apply(raw_span, tr, ti, gamma, state0, group,
                                            ops or CudaOps(), reduce_parameter_grads)
