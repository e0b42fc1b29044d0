"""Symmetric-memory (NVLink peer access) implementation of the ZeRO-1 collectives.

Set-up: the bf16 parameters of every sharded tensor and a full-shape bf16 gradient
accumulator for each of them are placed in two symmetric allocations
(``torch.distributed._symmetric_memory``: same layout on every rank, every rank's
copy mapped into every GPU).  A third small allocation holds epoch flags, the
gradient bucket of the small replicated parameters and the slots of the scalar
exchange.  The kernels are this package's own (``csrc/adam_step.cu`` PEERS variant,
``csrc/symm_ops.cu``); ``torch.distributed`` is used for bootstrap only.

Per optimizer step (epoch ``e``), for a sharded parameter ``p`` owned row-wise:

1. last micro-batch hook, main stream: accumulate into ``p``'s symmetric gradient,
   then store ``e`` into ``grad_flag[p][rank]`` on every rank;
2. optimizer stream: bounded wait until ``grad_flag[p][*] >= e`` locally, then
   * no clipping: one pass pulls the owned rows from all replicas, averages, runs
     Adam on the shard and pushes the new bf16 rows into all replicas;
   * clipping: one pass pulls and averages the rows into a local slice and reduces
     its squared norm; ``step()`` exchanges one scalar per rank, then the clip-fused
     Adam pass pushes the rows;
   then store ``e`` into ``param_flag[p][rank]`` on every rank;
3. before the next forward every rank waits (bounded) for all ``param_flag >= e``:
   all replicas are complete and nobody reads this rank's gradients any more.

Small replicated parameters are averaged in one bucket by the same pull kernel.
(reference: src/offload_adam/distributed_offload_adam.py:61-104, :182-306)
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _ext
from ..ops import grad_ops

_ALIGN = 256


def _round_up(x, a):
    return (x + a - 1) // a * a


class SymmZero1:
    def __init__(self, opt, model, timeout_ms=30000):
        import os

        # plain peer mappings only: no NVLS multicast binding for these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.opt = opt
        self.C = _ext.load(required=True)
        self.N = opt._world_size
        self.rank = opt._rank
        self.dev = opt.device
        self.timeout_ms = float(timeout_ms)
        if self.N > 8:
            raise RuntimeError("symmetric-memory path supports up to 8 ranks")
        if opt.grad_residency != "device":
            raise RuntimeError("symmetric-memory path needs grad_residency='device'")
        group = opt._pg
        self.group_name = group.group_name

        # ---- which tensors take this path
        # every offloaded dense tensor: row-sharded ones (pull own rows, push them back) and
        # replicated ones whose leading dimension does not divide (pull everything, every
        # rank steps its own replica with identical bits)
        self.params = [p for p in opt._offload_params if p not in opt._quant_params]
        self.is_sharded = {p: p in opt._sharded for p in self.params}
        self.index = {p: i for i, p in enumerate(self.params)}
        self.small = list(opt._inplace_entries)
        n_sym = len(self.params)

        # ---- layouts (identical on every rank)
        self.off = {}
        total = 0
        for p in self.params:
            self.off[p] = total
            total += _round_up(p.numel() * 2, _ALIGN)
        self.arena_bytes = max(total, _ALIGN)
        small_off, stotal = [], 0
        for e in self.small:
            small_off.append(stotal)
            stotal += _round_up(e["p"].numel() * 2, 32)
        self.small_bytes = max(stotal, 32)
        n_flags = 2 * n_sym * self.N + 4 * self.N
        self.ctrl_flag_words = _round_up(n_flags, 64)
        ctrl_bytes = self.ctrl_flag_words * 4 + _round_up(self.N * 4, _ALIGN) + self.small_bytes

        # ---- symmetric allocations + rendezvous
        self.param_arena = symm_mem.empty(self.arena_bytes, dtype=torch.uint8, device=self.dev)
        self.grad_arena = symm_mem.empty(self.arena_bytes, dtype=torch.uint8, device=self.dev)
        self.ctrl = symm_mem.empty(ctrl_bytes, dtype=torch.uint8, device=self.dev)
        self.ctrl.zero_()
        self.grad_arena.zero_()
        self.h_param = symm_mem.rendezvous(self.param_arena, group)
        self.h_grad = symm_mem.rendezvous(self.grad_arena, group)
        self.h_ctrl = symm_mem.rendezvous(self.ctrl, group)
        self.param_base = [int(x) for x in self.h_param.buffer_ptrs]
        self.grad_base = [int(x) for x in self.h_grad.buffer_ptrs]
        self.ctrl_base = [int(x) for x in self.h_ctrl.buffer_ptrs]

        # ---- views
        self.flags = self.ctrl[: self.ctrl_flag_words * 4].view(torch.int32)
        slots_off = self.ctrl_flag_words * 4
        self.slots = self.ctrl[slots_off: slots_off + self.N * 4].view(torch.float32)
        self.slots_off = slots_off
        self.small_off_bytes = slots_off + _round_up(self.N * 4, _ALIGN)
        self.small_sym = self.ctrl[self.small_off_bytes: self.small_off_bytes + self.small_bytes].view(torch.bfloat16)
        # flag regions (in words)
        self.F_GRAD = 0
        self.F_PARAM = n_sym * self.N
        self.F_SMALL_READY = 2 * n_sym * self.N
        self.F_SMALL_DONE = self.F_SMALL_READY + self.N
        self.F_SCALAR = self.F_SMALL_DONE + self.N

        # ---- move parameters into the symmetric arena, carve gradient views
        self.grad_view = {}
        for p in self.params:
            o, n = self.off[p], p.numel()
            home = self.param_arena[o: o + n * 2].view(torch.bfloat16).view(p.shape)
            home.copy_(p.data)
            p.data = home
            self.grad_view[p] = self.grad_arena[o: o + n * 2].view(torch.bfloat16).view(p.shape)
        self.acc_valid = {p: False for p in self.params}
        torch.cuda.empty_cache()  # the parameters' old storage goes back to the driver
        self.shard_bytes = {p: (p.numel() // self.N if self.is_sharded[p] else p.numel()) * 2
                            for p in self.params}
        # reduced gradient slices (clip path keeps them until step())
        self.red = {}
        if opt.max_grad_norm is not None:
            for p in self.params:
                shape = (p.shape[0] // self.N, *p.shape[1:]) if self.is_sharded[p] else p.shape
                self.red[p] = torch.empty(shape, dtype=torch.bfloat16, device=self.dev)

        # ---- small replicated parameters: accumulate in symmetric memory, step from a
        # local reduced copy
        self.small_red = torch.zeros(self.small_bytes // 2, dtype=torch.bfloat16, device=self.dev)
        for e, o in zip(self.small, small_off):
            n = e["p"].numel()
            sym_view = self.small_sym[o // 2: o // 2 + n].view(e["p"].shape)
            red_view = self.small_red[o // 2: o // 2 + n].view(e["p"].shape)
            opt.state[e["p"]]["grad"] = sym_view   # hooks accumulate here
            e["grad"] = red_view                    # the step reads (and zeroes) this
        opt._multi = None  # pointer table must be rebuilt with the new gradient views
        self.small_sq = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.small_reduced_epoch = 0

        # Status word of the bounded waits.  It lives in device memory: kernels poll it at
        # launch, and a word in host memory would make every launch wait for a PCIe read
        # queued behind the state DMA traffic.  The host sees it through an asynchronous
        # mirror refreshed at the end of every step.
        self.status = torch.zeros(4, dtype=torch.int32, device=self.dev)
        self.status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.local_sq = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.total_sq = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.epoch = 1
        # norm slots counted by this rank: its slices of sharded tensors, plus (rank 0
        # only) everything that is identical on all ranks
        idx = [opt._pid[p] for p in opt._all_params
               if p in opt._sharded or (self.rank == 0 and p not in opt._inplace_params)]
        self.norm_index = torch.tensor(idx, dtype=torch.int32, device=self.dev) if idx else None
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=group)

    # ------------------------------------------------------------ addressing
    def _flag_ptrs(self, region, word):
        """Address of flag ``word`` of ``region`` in every rank's control block."""
        return [b + 4 * (region + word) for b in self.ctrl_base]

    def _my_rows(self, base, p):
        """Address, in every rank's arena, of the part of ``p`` this rank reduces/updates."""
        first = self.rank * self.shard_bytes[p] if self.is_sharded[p] else 0
        return [b + self.off[p] + first for b in base]

    def handles(self, p):
        return p in self.index

    def _opt_stream(self):
        return self.opt._engine.opt_stream.cuda_stream

    # ------------------------------------------------------------------ hooks
    def accumulate(self, p, grad, sumsq=None):
        """Micro-batch gradient into the symmetric accumulator (main stream)."""
        acc = self.grad_view[p]
        if self.acc_valid[p]:
            grad_ops.grad_accumulate(acc, acc, grad, scratch=self.opt._scratch_main)
        else:
            acc.copy_(grad)
            self.acc_valid[p] = True

    @torch.no_grad()
    def grad_hook_last(self, p):
        opt, C, N = self.opt, self.C, self.N
        i = self.index[p]
        grad = opt._take_grad(p)
        self.accumulate(p, grad)
        self.acc_valid[p] = False  # the next step starts a fresh accumulator
        # announce: my replica of p's gradient is complete
        C.signal(self._flag_ptrs(self.F_GRAD, i * N + self.rank), self.epoch)
        eng = opt._engine
        eng.fork_from_main()
        s = self._opt_stream()
        C.wait_flags(self.flags, self.F_GRAD + i * N, N, self.epoch, self.timeout_ms, self.status,
                     C.SYMM_TIMEOUT_GRAD, s)
        if opt._step_in_backward:
            opt._step_offload(p, opt._param2group[p])
        else:
            C.peer_reduce(self.red[p], self._my_rows(self.grad_base, p), 1.0 / N, opt._slot(p),
                          eng.scratch, self.status, eng.max_ctas, s)
            opt._dev_grad[p] = self.red[p]

    def step_extra(self, p):
        """Extra arguments of the Adam pass of a sharded tensor."""
        kw = {"status": self.status}
        if self.is_sharded[p]:
            kw["p_peers"] = self._my_rows(self.param_base, p)
        if self.opt._step_in_backward:
            kw.update(g_peers=self._my_rows(self.grad_base, p), g_scale=1.0 / self.N)
        return kw

    def after_param_update(self, p):
        i = self.index[p]
        self.C.signal(self._flag_ptrs(self.F_PARAM, i * self.N + self.rank), self.epoch, self._opt_stream())

    # ------------------------------------------------------------ small bucket
    def reduce_small_bucket(self):
        """Average the small replicated gradients across ranks (one pull kernel)."""
        if not self.small or self.small_reduced_epoch == self.epoch:
            return
        C, N = self.C, self.N
        self.small_reduced_epoch = self.epoch
        C.signal(self._flag_ptrs(self.F_SMALL_READY, self.rank), self.epoch)
        C.wait_flags(self.flags, self.F_SMALL_READY, N, self.epoch, self.timeout_ms, self.status,
                     C.SYMM_TIMEOUT_GRAD)
        peers = [b + self.small_off_bytes for b in self.ctrl_base]
        want_sq = self.opt.max_grad_norm is not None
        C.peer_reduce(self.small_red, peers, 1.0 / N, self.small_sq if want_sq else None,
                      self.opt._scratch_main if want_sq else None, self.status)
        C.signal(self._flag_ptrs(self.F_SMALL_DONE, self.rank), self.epoch)

    # -------------------------------------------------------------- clip path
    def global_clip_coef(self):
        opt, C = self.opt, self.C
        self.reduce_small_bucket()
        opt._engine.join_main(wait_writeback=False)  # slice norms come from kernels on the optimizer stream
        extra = self.small_sq if (self.rank == 0 and self.small) else None
        grad_ops.clip_finalize(opt._normsq if self.norm_index is not None else None, self.norm_index,
                               extra, opt.max_grad_norm, total_sq=self.local_sq)
        C.scalar_exchange(self.local_sq, [b + self.slots_off for b in self.ctrl_base],
                          self._flag_ptrs(self.F_SCALAR, 0), self.slots,
                          self.flags[self.F_SCALAR: self.F_SCALAR + self.N], self.rank, self.epoch,
                          self.timeout_ms, self.status, self.total_sq)
        grad_ops.clip_finalize(None, None, self.total_sq, opt.max_grad_norm, coef_norm=opt._clip)
        return opt._clip[0:1]

    # ------------------------------------------------------------- step fences
    def before_finish(self):
        if self.opt._pending_inplace:
            self.reduce_small_bucket()

    def after_finish(self):
        """End of a step; the main stream is already ordered after the optimizer stream."""
        C, N = self.C, self.N
        if self.params:
            C.wait_flags(self.flags, self.F_PARAM, len(self.params) * N, self.epoch, self.timeout_ms,
                         self.status, C.SYMM_TIMEOUT_PARAM)
        if self.small and self.small_reduced_epoch == self.epoch:
            C.wait_flags(self.flags, self.F_SMALL_DONE, N, self.epoch, self.timeout_ms, self.status,
                         C.SYMM_TIMEOUT_PARAM)
            self.small_sym.zero_()
        self.epoch += 1
        self.check_status()
        # a kernel, not a DMA copy: a copy would queue behind the trailing state write-backs
        self.C.mirror_words(self.status, self.status_host)

    def check_status(self, blocking=False):
        """Raise if an earlier bounded wait gave up.  By default reads the host mirror
        written at the end of the previous step (no synchronisation)."""
        if blocking:
            self.status_host.copy_(self.status)
        code = int(self.status_host[0])
        if code != 0:
            names = {1: "a peer's gradient", 2: "a peer's parameter rows", 3: "the norm exchange"}
            raise RuntimeError(
                f"DistributedOffloadAdam[rank {self.rank}]: device-side wait for "
                f"{names.get(code, 'a peer')} timed out after {self.timeout_ms:.0f} ms; the step was "
                f"abandoned and optimizer state is no longer consistent across ranks")
