"""Symmetric-memory (NVLink peer access) implementation of the ZeRO-1 collectives.

Set-up: the bf16 parameters of every sharded dense tensor, the packed payload tensors of
every quantized weight and a full-shape bf16 gradient accumulator for each of them are
placed in symmetric allocations (``torch.distributed._symmetric_memory``: same layout on
every rank, every rank's copy mapped into every GPU).  A small control allocation holds
epoch flags, the gradient bucket of the small replicated parameters and the slots of the
scalar exchanges.  The kernels are this package's own (``csrc/adam_step.cu`` PEERS
variant, ``csrc/adam_quant.cu``, ``csrc/symm_ops.cu``); ``torch.distributed`` is used for
bootstrap only.

Per optimizer step (epoch ``e``), for a tensor ``p`` whose rows are divided among the ranks:

1. last micro-batch hook, main stream: accumulate into ``p``'s symmetric gradient,
   then store ``e`` into ``grad_flag[p][rank]`` on every rank;
2. optimizer stream: bounded wait until ``grad_flag[p][*] >= e`` locally, then
   * no clipping: one pass pulls the owned rows from all replicas, averages, runs
     Adam on the shard and pushes the new bf16 rows (a quantized weight: the re-quantized
     packed rows and their scales) into all replicas;
   * clipping: one pass pulls and averages the rows into a local slice and reduces
     its squared norm; ``step()`` exchanges one scalar per rank, then the clip-fused
     Adam pass pushes the rows;
   then store ``e`` into ``param_flag[p][rank]`` on every rank;
3. before the next forward every rank waits (bounded) for all ``param_flag >= e``:
   all replicas are complete and nobody reads this rank's gradients any more.

An NVFP4 weight needs max|master| of the whole updated weight before it can be
quantized: the Adam pass leaves the rank's maximum, one more scalar exchange (MAX)
combines them, and a second pass quantizes the rank's rows and pushes them.

``grad_layout='shard'`` replaces the full-shape accumulators by a two-slot exchange
window: every micro-batch's gradient of a tensor is copied into a slot, the ranks pull
and average their rows out of all replicas of the slot and add them to a shard-sized
accumulator; ready/done flags per slot and rank keep a slot from being overwritten
before every rank has read it.

Small replicated parameters are averaged in one bucket by the same pull kernel.
The first micro-batch's gradient is copied into the symmetric accumulator (one 4 B per
element pass, about 5 ms per step for an 8B model); adopting the autograd tensor
instead, as the single-GPU path does, would keep a second full-size gradient set alive
between the first two micro-batches.
(reference: src/offload_adam/distributed_offload_adam.py:61-104, :182-306)

Side effect of construction: ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` is set in the process
environment (unless already set) so that these buffers are plain peer mappings and are
never bound to an NVLink multicast object.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _ext
from ..ops import grad_ops

_ALIGN = 256
_WINDOW_SLOTS = 2


def _round_up(x, a):
    return (x + a - 1) // a * a


def _nbytes(t):
    return t.numel() * t.element_size()


def materialize_in_symmetric_memory(model, device, group=None, threshold=1024 * 1024, dtype=torch.bfloat16):
    """Give a model that was built on the ``meta`` device its storage, with every large
    parameter placed directly in a symmetric allocation.

    ``SymmZero1`` keeps the parameters of the peer-memory path in symmetric memory; a model
    that already exists in ordinary device memory is copied there, so for a moment both
    copies are alive.  A model whose weights fill most of the GPU (70B in bf16 is 141 GB of
    180) cannot afford that: build it with ``torch.device('meta')``, call this function, then
    initialise or load the weights and construct ``DistributedOffloadAdam(model,
    comm='symm', inplace_param_threshold=threshold)``, which recognises the allocation and
    adopts it.  Parameters with fewer than ``threshold`` elements get ordinary tensors (they
    are the ones the optimizer keeps on the GPU).  The contents are uninitialised.
    Collective: every rank of ``group`` must call it with the same model."""
    import os

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    seen, offsets, total = {}, {}, 0
    owners = []
    for module in model.modules():
        for name, p in list(module.named_parameters(recurse=False)):
            owners.append((module, name, p))
            if id(p) in seen or p.numel() < threshold:
                continue
            seen[id(p)] = p
            offsets[id(p)] = total
            total += _round_up(p.numel() * 2, _ALIGN)
    arena = symm_mem.empty(max(total, _ALIGN), dtype=torch.uint8, device=device)
    handle = symm_mem.rendezvous(arena, group)
    new = {}
    for module, name, p in owners:
        if id(p) not in new:
            if id(p) in offsets:
                o = offsets[id(p)]
                data = arena[o: o + p.numel() * 2].view(dtype).view(p.shape)
            else:
                data = torch.empty(p.shape, dtype=dtype, device=device)
            new[id(p)] = torch.nn.Parameter(data, requires_grad=p.requires_grad)
        setattr(module, name, new[id(p)])  # shared (tied) parameters stay shared
    for module in model.modules():
        for name, b in list(module.named_buffers(recurse=False)):
            if b is not None and b.is_meta:
                setattr(module, name, torch.empty(b.shape, dtype=b.dtype, device=device))
    model._oab_symmetric_params = {"arena": arena, "handle": handle, "group": group,
                                   "offsets": {id(new[k]): v for k, v in offsets.items()}}
    return model


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
        self.shard_layout = opt.grad_layout == "shard"
        N = self.N

        # ---- which tensors take this path
        # every offloaded dense tensor: row-sharded ones (pull own rows, push them back) and
        # replicated ones whose leading dimension does not divide (pull everything, every
        # rank steps its own replica with identical bits); quantized weights when the fused
        # Adam + re-quantize + push kernels take their shape
        self.params = [p for p in opt._offload_params
                       if p not in opt._quant_params or opt._fused_quant_ok(p)]
        self.is_quant = {p: p in opt._quant_params for p in self.params}
        self.is_sharded = {p: p in opt._sharded for p in self.params}
        self.index = {p: i for i, p in enumerate(self.params)}
        self.small = list(opt._inplace_entries)
        n_sym = len(self.params)

        # ---- layouts (identical on every rank)
        # gradient arena: a full-shape bf16 accumulator per tensor ('shard' layout: only
        # for the tensors whose rows do not divide, the others go through the window)
        self.goff, gtotal = {}, 0
        for p in self.params:
            if self.shard_layout and self.is_sharded[p]:
                continue
            self.goff[p] = gtotal
            gtotal += _round_up(p.numel() * 2, _ALIGN)
        # parameter arena: bf16 data of dense tensors, both payload tensors of quantized ones
        self.poff, ptotal = {}, 0
        for p in self.params:
            if self.is_quant[p]:
                offs = []
                for name in p.KERNEL_PAYLOAD:
                    offs.append(ptotal)
                    ptotal += _round_up(_nbytes(getattr(p, name)), _ALIGN)
                self.poff[p] = tuple(offs)
            else:
                self.poff[p] = ptotal
                ptotal += _round_up(p.numel() * 2, _ALIGN)
        self.window_bytes = 0
        if self.shard_layout:
            biggest = max((p.numel() * 2 for p in self.params if self.is_sharded[p]), default=0)
            self.window_bytes = _round_up(biggest, _ALIGN)
        small_off, stotal = [], 0
        for e in self.small:
            small_off.append(stotal)
            stotal += _round_up(e["p"].numel() * 2, 32)
        self.small_bytes = max(stotal, 32)
        # flag regions (in words)
        self.F_GRAD = 0
        self.F_PARAM = n_sym * N
        self.F_SMALL_READY = 2 * n_sym * N
        self.F_SMALL_DONE = self.F_SMALL_READY + N
        self.F_SCALAR = self.F_SMALL_DONE + N          # 4 sets of N: {main, optimizer stream} x {even, odd}
        self.F_WIN_READY = self.F_SCALAR + 4 * N       # per window slot and rank
        self.F_WIN_DONE = self.F_WIN_READY + _WINDOW_SLOTS * N
        n_flags = self.F_WIN_DONE + _WINDOW_SLOTS * N
        self.ctrl_flag_words = _round_up(n_flags, 64)
        self.slots_off = self.ctrl_flag_words * 4
        self.small_off_bytes = self.slots_off + _round_up(4 * N * 4, _ALIGN)
        ctrl_bytes = self.small_off_bytes + self.small_bytes

        # ---- symmetric allocations + rendezvous
        # a model materialised by materialize_in_symmetric_memory already lives in an
        # allocation of exactly this layout: adopt it instead of copying the parameters
        pre = getattr(model, "_oab_symmetric_params", None)
        adopted = (pre is not None and pre["group"] is group and pre["arena"].numel() >= max(ptotal, _ALIGN)
                   and not any(self.is_quant.values())
                   and all(pre["offsets"].get(id(p)) == self.poff[p] for p in self.params))
        self.param_arena = pre["arena"] if adopted else \
            symm_mem.empty(max(ptotal, _ALIGN), dtype=torch.uint8, device=self.dev)
        self.grad_arena = symm_mem.empty(max(gtotal, _ALIGN), dtype=torch.uint8, device=self.dev)
        self.ctrl = symm_mem.empty(ctrl_bytes, dtype=torch.uint8, device=self.dev)
        self.ctrl.zero_()
        self.grad_arena.zero_()
        self.h_param = pre["handle"] if adopted else symm_mem.rendezvous(self.param_arena, group)
        self.h_grad = symm_mem.rendezvous(self.grad_arena, group)
        self.h_ctrl = symm_mem.rendezvous(self.ctrl, group)
        self.param_base = [int(x) for x in self.h_param.buffer_ptrs]
        self.grad_base = [int(x) for x in self.h_grad.buffer_ptrs]
        self.ctrl_base = [int(x) for x in self.h_ctrl.buffer_ptrs]
        self.window = None
        if self.window_bytes:
            self.window = symm_mem.empty(_WINDOW_SLOTS * self.window_bytes, dtype=torch.uint8, device=self.dev)
            self.h_window = symm_mem.rendezvous(self.window, group)
            self.window_base = [int(x) for x in self.h_window.buffer_ptrs]
        self.window_use = 0

        # ---- views
        self.flags = self.ctrl[: self.ctrl_flag_words * 4].view(torch.int32)
        self.slots = self.ctrl[self.slots_off: self.slots_off + 4 * N * 4].view(torch.float32)
        self.small_sym = self.ctrl[self.small_off_bytes: self.small_off_bytes + self.small_bytes].view(torch.bfloat16)

        # ---- move parameters (payloads) into the symmetric arena, carve gradient views
        self.grad_view = {}
        for p in self.params:
            if self.is_quant[p]:
                for name, o in zip(p.KERNEL_PAYLOAD, self.poff[p]):
                    t = getattr(p, name)
                    home = self.param_arena[o: o + _nbytes(t)].view(t.dtype).view(t.shape)
                    home.copy_(t)
                    setattr(p, name, home)  # p.data is rebuilt from these attributes on every access
            elif not adopted:
                o, n = self.poff[p], p.numel()
                home = self.param_arena[o: o + n * 2].view(torch.bfloat16).view(p.shape)
                home.copy_(p.data)
                p.data = home
            if p in self.goff:
                o, n = self.goff[p], p.numel()
                self.grad_view[p] = self.grad_arena[o: o + n * 2].view(torch.bfloat16).view(p.shape)
        self.adopted_param_arena = adopted
        self.acc_valid = {p: False for p in self.params}
        torch.cuda.empty_cache()  # the parameters' old storage goes back to the driver
        self.shard_bytes = {p: (p.numel() // N if self.is_sharded[p] else p.numel()) * 2 for p in self.params}
        # reduced gradient slices: the clip path keeps them until step(), the 'shard' layout
        # accumulates the micro-batches in them
        self.red = {}
        for p in self.params:
            if opt.max_grad_norm is not None or (self.shard_layout and self.is_sharded[p]):
                shape = (p.shape[0] // N, *p.shape[1:]) if self.is_sharded[p] else tuple(p.shape)
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
        self.xseq = [1, 1]   # sequence numbers of the scalar exchanges: main stream, optimizer stream
        self._params_signaled = False
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

    def _my_rows(self, base, off, p):
        """Address, in every rank's arena, of the part of ``p`` this rank reduces/updates."""
        first = self.rank * self.shard_bytes[p] if self.is_sharded[p] else 0
        return [b + off + first for b in base]

    def handles(self, p):
        return p in self.index

    def _opt_stream(self):
        return self.opt._engine.opt_stream.cuda_stream

    def quant_replicas(self, p):
        """``(row0, payload0 addresses, payload1 addresses)`` of quantized weight ``p``: this
        rank's first row and the base of both payload tensors in every replica it stores
        into (all ranks' when the rows are divided, its own otherwise)."""
        o0, o1 = self.poff[p]
        if self.is_sharded[p]:
            row0 = self.rank * (p.shape[0] // self.N)
            return row0, [b + o0 for b in self.param_base], [b + o1 for b in self.param_base]
        return 0, [self.param_base[self.rank] + o0], [self.param_base[self.rank] + o1]

    # ------------------------------------------------------------------ hooks
    def accumulate(self, p, grad, sumsq=None):
        """Micro-batch gradient into the symmetric accumulator (main stream)."""
        acc = self.grad_view[p]
        if self.acc_valid[p]:
            grad_ops.grad_accumulate(acc, acc, grad, scratch=self.opt._scratch_main)
        else:
            acc.copy_(grad)
            self.acc_valid[p] = True

    def windowed(self, p):
        return self.shard_layout and self.is_sharded[p]

    @torch.no_grad()
    def grad_hook_window(self, p, last):
        """``grad_layout='shard'``: this micro-batch's gradient goes through the exchange
        window; the mean of this rank's rows over the ranks is added to its shard-sized
        accumulator."""
        opt, C, N = self.opt, self.C, self.N
        grad = opt._take_grad(p)
        u = self.window_use
        self.window_use += 1
        slot = u % _WINDOW_SLOTS
        if u >= _WINDOW_SLOTS:
            # every rank has finished reading what this slot held before
            C.wait_flags(self.flags, self.F_WIN_DONE + slot * N, N, u - _WINDOW_SLOTS + 1, self.timeout_ms,
                         self.status, C.SYMM_TIMEOUT_GRAD)
        nbytes = p.numel() * 2
        off = slot * self.window_bytes
        self.window[off: off + nbytes].view(torch.bfloat16).view(p.shape).copy_(grad)
        C.signal(self._flag_ptrs(self.F_WIN_READY, slot * N + self.rank), u + 1)
        eng = opt._engine
        eng.fork_from_main()
        s = self._opt_stream()
        C.wait_flags(self.flags, self.F_WIN_READY + slot * N, N, u + 1, self.timeout_ms, self.status,
                     C.SYMM_TIMEOUT_GRAD, s)
        red = self.red[p]
        first = opt._dev_grad.get(p) is None
        want_sq = last and opt.max_grad_norm is not None
        C.peer_reduce(red, [b + off + self.rank * self.shard_bytes[p] for b in self.window_base], 1.0 / N,
                      opt._slot(p) if want_sq else None, eng.scratch if want_sq else None, self.status,
                      eng.max_ctas, s, None if first else red)
        C.signal(self._flag_ptrs(self.F_WIN_DONE, slot * N + self.rank), u + 1, s)
        opt._dev_grad[p] = red
        if last and opt._step_in_backward:
            opt._step_offload(p, opt._param2group[p])

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
            C.peer_reduce(self.red[p], self._my_rows(self.grad_base, self.goff[p], p), 1.0 / N, opt._slot(p),
                          eng.scratch, self.status, eng.max_ctas, s)
            opt._dev_grad[p] = self.red[p]

    def step_extra(self, p):
        """Extra arguments of the Adam pass of a tensor on this path."""
        kw = {"status": self.status}
        if self.is_sharded[p] and not self.is_quant[p]:
            kw["p_peers"] = self._my_rows(self.param_base, self.poff[p], p)
        if self.opt._step_in_backward and not self.windowed(p):
            kw.update(g_peers=self._my_rows(self.grad_base, self.goff[p], p), g_scale=1.0 / self.N)
        return kw

    def after_param_update(self, p):
        """The rows of ``p`` are in every replica once the kernels enqueued so far have run; the
        flags of all tensors are raised together at the end of the step (``before_finish``):
        nobody waits for a single tensor, and one launch replaces one per tensor."""

    # ------------------------------------------------------------ scalar exchanges
    def _exchange(self, value, out, on_opt_stream, op_max):
        """All-reduce of one fp32 scalar through the flag slots.  Exchanges of one stream
        alternate between two sets of slots and carry increasing sequence numbers."""
        which = 1 if on_opt_stream else 0
        k = self.xseq[which]
        self.xseq[which] = k + 1
        s = 2 * which + (k & 1)
        N = self.N
        self.C.scalar_exchange(value, [b + self.slots_off + 4 * s * N for b in self.ctrl_base],
                               self._flag_ptrs(self.F_SCALAR, s * N), self.slots[s * N: (s + 1) * N],
                               self.flags[self.F_SCALAR + s * N: self.F_SCALAR + (s + 1) * N], self.rank, k,
                               self.timeout_ms, self.status, out,
                               self._opt_stream() if on_opt_stream else 0, op_max)

    def combine_amax(self, local_amax, tensor_amax):
        """max|master| of a row-divided NVFP4 weight over all ranks (optimizer stream)."""
        self._exchange(local_amax, tensor_amax, True, True)

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
        opt = self.opt
        self.reduce_small_bucket()
        opt._engine.join_main(wait_writeback=False)  # slice norms come from kernels on the optimizer stream
        extra = self.small_sq if (self.rank == 0 and self.small) else None
        grad_ops.clip_finalize(opt._normsq if self.norm_index is not None else None, self.norm_index,
                               extra, opt.max_grad_norm, total_sq=self.local_sq)
        self._exchange(self.local_sq, self.total_sq, False, False)
        grad_ops.clip_finalize(None, None, self.total_sq, opt.max_grad_norm, coef_norm=opt._clip)
        return opt._clip[0:1]

    # ------------------------------------------------------------- step fences
    def before_finish(self):
        if self.opt._pending_inplace:
            self.reduce_small_bucket()
        if self.params and self.opt._step_dirty:
            # every parameter kernel of this step is on the optimizer stream by now: raise this
            # rank's flag of every tensor on every rank (a tensor that got no gradient was not
            # stepped on any rank; its flag goes up with the others so that nobody waits for it)
            self.C.signal_many([b for b in self.ctrl_base], self.F_PARAM + self.rank, self.N, len(self.params),
                               self.epoch, self._opt_stream())
            self._params_signaled = True

    def after_finish(self):
        """End of a step; the main stream is already ordered after the optimizer stream."""
        C, N = self.C, self.N
        if self.params:
            if not self._params_signaled:  # only small parameters were stepped
                C.signal_many([b for b in self.ctrl_base], self.F_PARAM + self.rank, N, len(self.params), self.epoch)
            self._params_signaled = False
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
            names = {1: "a peer's gradient", 2: "a peer's parameter rows", 3: "a scalar exchange"}
            raise RuntimeError(
                f"DistributedOffloadAdam[rank {self.rank}]: device-side wait for "
                f"{names.get(code, 'a peer')} timed out after {self.timeout_ms:.0f} ms; the step was "
                f"abandoned and optimizer state is no longer consistent across ranks")
