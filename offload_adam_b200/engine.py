"""Transfer layer of the offloaded optimizers.

``TransferEngine`` owns the side streams and hides *how* optimizer state that
lives in pinned host memory meets the gradient on the GPU:

``zero_copy``  the step kernel reads and writes the mapped host buffers itself,
               over PCIe, in one launch per tensor; no staging memory.
``staged``     the C++ copy engine (csrc/offload_engine.cpp) cuts a tensor into
               chunks and pipelines H2D -> kernel -> D2H through a circular
               staging buffer in device memory on three streams; helper threads
               load the next step's state ahead of time and issue the
               write-backs.
``host``       CPU tensors: everything is synchronous PyTorch (unit tests,
               gloo multi-process tests).

All work is enqueued on side streams ordered after the main stream's current
position; nothing blocks the host except the bounded back-pressure on queued
gradient bytes.  The reference does the same job with whole-tensor
``.to(device)`` / ``copy_`` calls on two streams plus per-parameter events
(reference: src/offload_adam/offload_adam.py:344-382).
"""

from __future__ import annotations

import collections

import torch

from . import _ext
from .ops import grad_ops
from .ops.adam_step import adam_step
from .ops.oracle import MODE_IDS, beta_hat


class TransferEngine:
    def __init__(self, device, mode, n_tensors, transfer="auto", chunk_elems=8 << 20, ring_slots=4,
                 max_ctas=0, max_inflight_bytes=8 << 30, staging_bytes=0, async_writeback=True,
                 serialize=False, canaries=False, lazy_resident=False):
        self.device = torch.device(device)
        self.mode = mode
        self.mode_id = MODE_IDS[mode]
        self.cuda = self.device.type == "cuda"
        if not self.cuda:
            transfer = "host"
        elif transfer == "auto":
            # measured on B200 over PCIe 5 x16: DMA through the staging buffer sustains ~45 GB/s
            # per direction for the step, the zero-copy kernel ~16-40 GB/s
            transfer = "staged"
        if transfer not in ("zero_copy", "staged", "host"):
            raise ValueError(f"transfer must be 'auto', 'zero_copy' or 'staged' (got {transfer!r})")
        self.transfer = transfer
        self.max_ctas = int(max_ctas)
        self.max_inflight_bytes = int(max_inflight_bytes)
        self._inflight = collections.deque()  # (event, nbytes)
        self._inflight_bytes = 0
        self.h2d_stream = self.d2h_stream = self.opt_stream = None
        self._native = None
        # debugging aid: every transfer and step completes before the call returns, no
        # helper threads, no early loads; results must equal the overlapped run bit for bit
        self.serialize = bool(serialize)
        if self.serialize:
            async_writeback = False
        self.chunk_elems = int(chunk_elems)
        self._marks, self._last_marks = [], []
        self.scratch = None
        self.staging_bytes = 0
        self._ring_floor_extra = 0
        if self.cuda:
            self.C = _ext.load(required=True)
            with torch.cuda.device(self.device):
                self.opt_stream = torch.cuda.Stream()
                self.h2d_stream = torch.cuda.Stream()
                self.d2h_stream = torch.cuda.Stream()
                self.scratch = grad_ops.sumsq_scratch(self.device)
                if transfer == "staged":
                    # circular staging buffer: pipelines the chunks of a step and doubles as
                    # the early-H2D / trailing-D2H area
                    chunk_elems = max(16, int(chunk_elems) // 16 * 16)
                    # smallest ring that pipelines a step: the engine's floor plus `ring_slots`
                    # full-width chunks.  `staging_bytes` comes on top of it: that part buys
                    # overlap (early loads, trailing write-backs) or residency.
                    floor = self.C.OffloadEngine.min_ring_bytes(chunk_elems)
                    self.chunk_elems = chunk_elems
                    self._ring_floor_extra = int(ring_slots) * chunk_elems * 10
                    smallest = (floor + self._ring_floor_extra + 255) // 256 * 256
                    nbytes = (smallest + max(0, int(staging_bytes)) + 255) // 256 * 256
                    while True:
                        # the buffer only buys overlap: when memory is short, take less
                        try:
                            ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
                            break
                        except torch.cuda.OutOfMemoryError:
                            if nbytes <= smallest:
                                raise
                            nbytes = max(smallest, nbytes // 2 // 256 * 256)
                    self.staging_bytes = nbytes
                    self._native = self.C.OffloadEngine(
                        self.device.index or 0, self.opt_stream.cuda_stream,
                        self.h2d_stream.cuda_stream, self.d2h_stream.cuda_stream, ws,
                        chunk_elems, self.max_ctas, n_tensors, bool(async_writeback), bool(canaries),
                        bool(lazy_resident),
                    )

    # ------------------------------------------------------------ stream glue
    def fork_from_main(self):
        """Side work enqueued after this call starts after everything already on
        the main stream."""
        if self.cuda:
            self.opt_stream.wait_stream(torch.cuda.current_stream(self.device))

    def join_main(self, wait_writeback=True):
        """The main stream waits for the side-stream work enqueued so far.  With
        ``wait_writeback=False`` it waits for the kernels only (parameters updated); the
        D2H write-back of the state may still be in flight and is ordered before any
        later H2D of the same tensor by the engine."""
        if not self.cuda:
            return
        main = torch.cuda.current_stream(self.device)
        if self._native is not None:
            if wait_writeback:
                self._native.join(main.cuda_stream)
            else:
                self._native.join_compute(main.cuda_stream)
        else:
            main.wait_stream(self.opt_stream)

    # ----------------------------------------------------------------- tracing
    def mark(self, name, which="main"):
        """Record a named timing event on one of the engine's streams (``'main'`` |
        ``'opt'`` | ``'h2d'`` | ``'d2h'``).  Marks cost one event record each and are only
        taken when the optimizer runs with ``verbose`` > 2; ``trace_report`` turns them
        into milliseconds relative to the first mark of the step."""
        if not self.cuda:
            return
        stream = {"main": torch.cuda.current_stream(self.device), "opt": self.opt_stream,
                  "h2d": self.h2d_stream, "d2h": self.d2h_stream}[which]
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream)
        self._marks.append((name, which, ev))

    def begin_trace(self):
        """Start a new trace; the previous one stays readable until then."""
        self._last_marks, self._marks = self._marks, []

    def trace_report(self, current=True):
        """``{name@stream: ms since the first mark}`` of the current (or previous) trace;
        ``None`` while some of its events have not completed.  Never blocks."""
        marks = self._marks if current else self._last_marks
        if not marks or not all(ev.query() for _, _, ev in marks):
            return None
        t0 = marks[0][2]
        return {f"{name}@{which}": round(t0.elapsed_time(ev), 3) for name, which, ev in marks}

    def start_prefetch(self, items, max_inflight=2):
        """Hand a plan of early loads to the engine's helper thread: ``items`` is a list
        of ``(pid, states, chunk)`` in the order the tensors will be stepped (``chunk``: the
        tensor's own chunk length in elements, 0 for the engine's).  The thread keeps
        ``max_inflight`` chunk copies outstanding until the staging buffer is full."""
        if self._native is None or not items:
            return
        plan = [(pid, st["exp_avg"], st["exp_avg_sq"], st.get("master_params", st.get("rounding_error")),
                 int(chunk)) for pid, st, chunk in items]
        self._native.start_prefetch(self.mode_id, plan, int(max_inflight))

    def wait_writeback(self):
        """Block the host until the state of every step enqueued so far is back in host
        memory; early loads keep running."""
        if not self.cuda:
            return
        if self._native is not None:
            self._native.wait_writebacks()
        else:
            self.opt_stream.synchronize()

    def invalidate_prefetched(self):
        """The caller is about to change host state behind the engine's back (resume,
        master reload): wait for everything in flight and drop what was loaded early."""
        self.synchronize()
        if self._native is not None:
            self._native.discard_prefetched()

    def stop_prefetch(self):
        if self._native is not None:
            self._native.stop_prefetch()

    @property
    def can_prefetch(self):
        return self._native is not None and not self.serialize

    def make_resident(self, pid, n):
        """Give tensor ``pid`` (``n`` elements of state) a permanent place at the front of
        the staging buffer: loaded once, stepped with one launch, written back after
        every step, never loaded again.  Only before the first step or early load.
        Returns False when it does not fit."""
        if self._native is None:
            return False
        return bool(self._native.make_resident(int(pid), self.mode_id, int(n)))

    @property
    def can_make_resident(self):
        return self._native is not None

    def resident_budget(self, state_bytes):
        """Bytes of the staging buffer that resident tensors may take when the optimizer's
        state is ``state_bytes`` in all: everything when it fits next to the smallest
        ring, else all but a ring of an eighth of the buffer (at most 4 GiB), through
        which the other tensors stream."""
        if self._native is None:
            return 0
        floor = self.C.OffloadEngine.min_ring_bytes(self.chunk_elems) + self._ring_floor_extra
        have = self.staging_bytes
        if state_bytes + floor <= have:
            return have - floor
        ring = max(floor, min(4 << 30, have // 8))
        return max(0, have - ring)

    def wait_host_grad(self, pid):
        """Order later work of the optimizer stream after the last copy of tensor ``pid``'s
        gradient into its host buffer (callers whose kernels read that buffer directly)."""
        if self._native is not None:
            self._native.wait_host_grad(int(pid))

    def is_resident(self, pid):
        return self._native is not None and self._native.is_resident(int(pid))

    @property
    def resident_bytes(self):
        return int(self._native.resident_bytes()) if self._native is not None else 0

    def prefetch(self, pid, states, host_grad=None, from_off=0, max_chunks=0, max_inflight=0, chunk=0):
        """Start the H2D of a tensor's state ahead of its step (staged transfer only),
        at most ``max_chunks`` chunks of it (0: as many as fit).  Returns
        ``(offset, full)``: the element offset up to which the tensor is loaded and
        whether the staging buffer refused the next chunk.  ``max_inflight`` > 0 issues nothing while that
        many earlier prefetch copies are still running."""
        n = states["exp_avg"].numel()
        if self._native is None:
            return n, False
        extra = states.get("master_params", states.get("rounding_error"))
        return self._native.prefetch(pid, self.mode_id, host_grad, states["exp_avg"],
                                     states["exp_avg_sq"], extra, int(from_off), int(max_chunks),
                                     int(max_inflight), int(chunk))

    def synchronize(self):
        """Block the host until everything enqueued so far has finished, including
        write-backs the helper thread has not issued yet.  Stops the early loads."""
        if self.cuda:
            if self._native is not None:
                self._native.synchronize()
            self.opt_stream.synchronize()
            self.h2d_stream.synchronize()
            self.d2h_stream.synchronize()

    def _retain(self, tensor, copied_out=False):
        """Keep a main-stream tensor alive until the side streams are done with it
        and apply back-pressure on the bytes queued behind PCIe.  ``copied_out``: the
        tensor is also the source of a D2H copy (not only read by kernels)."""
        if not self.cuda or tensor is None:
            return
        tensor.record_stream(self.opt_stream)
        via_d2h = copied_out and self._native is not None
        if via_d2h:
            tensor.record_stream(self.d2h_stream)
        nbytes = tensor.numel() * tensor.element_size()
        ev = torch.cuda.Event()
        # kernels consume gradients on the optimizer stream; trailing state write-backs on
        # the D2H stream must not count against the gradient budget
        ev.record(self.d2h_stream if via_d2h else self.opt_stream)
        self._inflight.append((ev, nbytes))
        self._inflight_bytes += nbytes
        while self._inflight and (self._inflight[0][0].query() or
                                  self._inflight_bytes > self.max_inflight_bytes):
            ev0, n0 = self._inflight.popleft()
            if not ev0.query():
                ev0.synchronize()
            self._inflight_bytes -= n0

    # --------------------------------------------------------------- gradient
    def grad_to_host(self, pid, host_grad, dev_grad, first, sumsq=None):
        """host_grad = dev_grad (first) or bf16(host_grad + dev_grad); optional sum of
        squares of the result into ``sumsq`` (fp32 scalar on the device)."""
        if not self.cuda:
            grad_ops.grad_accumulate(host_grad, dev_grad, None if first else host_grad, sumsq=sumsq)
            return
        self.fork_from_main()
        if self._native is not None:
            self._native.staged_grad_to_host(pid, host_grad, dev_grad, first, sumsq, self.scratch)
        else:
            s = self.opt_stream.cuda_stream
            if first and sumsq is None:
                with torch.cuda.stream(self.opt_stream):
                    host_grad.copy_(dev_grad, non_blocking=True)
            else:
                grad_ops.grad_accumulate(host_grad, dev_grad, None if first else host_grad,
                                         sumsq=sumsq, scratch=self.scratch, max_ctas=self.max_ctas,
                                         stream=s, use_cuda=True)
        self._retain(dev_grad, copied_out=True)
        if self.serialize:
            self.synchronize()

    # ------------------------------------------------------------------- step
    def step(self, pid, param, dev_grad, host_grad, states, hp, step, decoupled, clip=None, seed=0,
             amax=None, fork=True, g_peers=None, g_scale=1.0, p_peers=None, status=None, quant=None,
             chunk=0, master_copy=None, retain=True):
        """Adam step of one offloaded tensor (or shard).

        ``states`` holds the host tensors ``exp_avg``, ``exp_avg_sq`` and, by mode,
        ``master_params`` / ``rounding_error``.  The gradient is ``dev_grad``,
        ``host_grad`` or bf16(dev_grad + host_grad), or (``g_peers``: peer-mapped
        addresses of the same rows in every rank's replica) the rank-ordered average
        pulled over NVLink.  ``p_peers`` makes the kernel store the updated bf16 rows
        into every replica.  ``param`` may be None when no bf16 write-back is wanted
        (fp32_master only).

        ``quant`` (a ``_C.QuantSpec``; staged transfer only) re-quantizes the updated
        master and stores the packed rows into every replica named by the spec in the same
        pass; ``chunk`` is then the tensor's chunk length (whole rows).  For NVFP4, whose
        tensor scale needs the whole updated weight, the pass only leaves max|master| in
        ``amax`` and the updated master on the device (in ``master_copy`` unless the tensor
        is resident); the address to quantize from is returned.
        """
        lr, wd, beta1, beta2, eps = hp
        if self.cuda and fork:
            self.fork_from_main()
        if self._native is not None:
            extra = states.get("master_params", states.get("rounding_error"))
            where = self._native.staged_step(
                pid, self.mode_id, param, dev_grad, host_grad, states["exp_avg"],
                states["exp_avg_sq"], extra, float(lr), float(wd), beta_hat(beta1, step),
                beta_hat(beta2, step), float(eps), bool(decoupled), clip, int(seed), 0, amax,
                list(g_peers or ()), float(g_scale), list(p_peers or ()), status, int(chunk), quant,
                master_copy,
            )
        else:
            if quant is not None:
                raise RuntimeError("fused re-quantization needs transfer='staged'")
            where = 0
            st = dict(states)
            if dev_grad is not None:
                st["grad"], g2 = dev_grad, host_grad
            else:
                st["grad"], g2 = host_grad, None  # both None: the gradient comes from g_peers
            adam_step(
                self.mode_id, param, st, lr, wd, beta1, beta2, eps, step,
                decoupled_weight_decay=decoupled, seed=seed, clip_coef=clip, grad2=g2, amax=amax,
                max_ctas=self.max_ctas,
                stream=self.opt_stream.cuda_stream if self.cuda else 0,
                use_cuda=self.cuda, g_peers=g_peers, g_scale=g_scale, p_peers=p_peers, status=status,
            )
        if retain:
            self._retain(dev_grad)
        if self.serialize:
            self.synchronize()
        return where

    def bytes_moved(self):
        if self._native is not None:
            return self._native.bytes_h2d(), self._native.bytes_d2h()
        return None
