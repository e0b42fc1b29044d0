"""``DistributedOffloadAdam``: ZeRO-1 on top of ``OffloadAdam``.

Parameters are replicated on every rank; the optimizer state of every large
parameter whose leading dimension divides by the world size is sharded by rows,
so each rank keeps (and streams over PCIe) ``1/world`` of the moments and of the
fp32 master.  On the last micro-batch the gradient of a sharded parameter is
reduce-scattered (average), the owning rank updates its row slice and the
updated slices are all-gathered into every replica.  Small parameters and
parameters that do not divide are replicated and all-reduced
(reference: src/offload_adam/distributed_offload_adam.py:1-314).

Two communication back ends implement those three collectives:

``comm='nccl'``  ``torch.distributed`` collectives (NCCL on GPUs, gloo on CPU).
                 This is the baseline path and the one CPU tests exercise.
``comm='symm'``  the parameters and the gradient accumulators live in symmetric
                 memory; one kernel per parameter pulls the peers' gradient rows
                 over NVLink, averages them, runs Adam on the shard and pushes
                 the new bf16 rows (for a quantized weight: the re-quantized packed
                 rows) into every replica (``parallel/symm.py``, ``csrc/symm_ops.cu``,
                 ``csrc/adam_step.cu``, ``csrc/adam_quant.cu``).  No NCCL call on that path.
``comm='auto'``  ``symm`` on CUDA with world size > 1 when symmetric memory can
                 be set up, else ``nccl``.

Reductions accumulate in fp32 over the ranks' bf16 gradients in rank order and
round once to bf16, on both back ends.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..offload_adam import OffloadAdam
from ..ops import grad_ops


class DistributedOffloadAdam(OffloadAdam):
    """Sharded-state (ZeRO-1) variant of :class:`OffloadAdam`.

    Extra keyword-only arguments: ``process_group`` (default: the world group),
    ``comm`` (``'auto'`` | ``'nccl'`` | ``'symm'``), ``wait_timeout_ms`` (bound
    of every device-side wait on a peer in the ``symm`` path) and ``grad_layout``:

    * ``'full'`` (default, the reference's layout): every rank accumulates the whole
      gradient over the micro-batches and the ranks are averaged once, on the last one;
    * ``'shard'``: every micro-batch's gradient of a sharded tensor is averaged over the
      ranks at once and only this rank's rows are accumulated.  Accumulators (in HBM or
      in pinned host memory, by ``grad_residency``) shrink by the world size, which is
      what lets a model whose full-shape gradient does not fit next to its weights (70B
      on 8 GPUs) train at all; the price is one reduce-scatter per tensor and
      micro-batch, and a different rounding order (mean over ranks first, then the bf16
      sum over micro-batches).  With ``comm='symm'`` the reduce-scatter is a pull out of a
      two-slot exchange window in symmetric memory (``parallel/symm.py``), with
      ``comm='nccl'`` a ``reduce_scatter_tensor``.

    With ``seed=None`` rank 0 draws the seed of the stochastic-rounding stream and
    broadcasts it: replicated tensors are stepped on every rank and must round alike.
    """

    def __init__(self, model, *, process_group=None, comm="auto", wait_timeout_ms=30000,
                 grad_layout="full", **kwargs):
        if not dist.is_available() or not dist.is_initialized():
            raise RuntimeError(
                "DistributedOffloadAdam requires torch.distributed to be initialized; "
                "call dist.init_process_group first."
            )
        if comm not in ("auto", "nccl", "symm"):
            raise ValueError(f"comm must be 'auto', 'nccl' or 'symm' (got {comm!r})")
        if grad_layout not in ("full", "shard"):
            raise ValueError(f"grad_layout must be 'full' or 'shard' (got {grad_layout!r})")
        self.grad_layout = grad_layout
        self._pg = process_group if process_group is not None else dist.group.WORLD
        self._world_size = dist.get_world_size(self._pg)
        self._rank = dist.get_rank(self._pg)
        self._sharded = set()
        self._requested_comm = comm
        self._wait_timeout_ms = int(wait_timeout_ms)
        self._symm = None
        self.comm = "nccl"
        super().__init__(model, **kwargs)
        self._setup_comm(model)

    # --------------------------------------------------------------- sharding
    def _is_sharded_shape(self, p):
        return (self._world_size > 1 and p.dim() >= 1 and p.shape[0] % self._world_size == 0
                and p not in self._inplace_params)

    def _rows(self, p):
        ds = p.shape[0] // self._world_size
        return self._rank * ds, (self._rank + 1) * ds

    def _shard_slice(self, p):
        """This rank's row slice of the bf16 parameter (a view)."""
        lo, hi = self._rows(p)
        return p.data[lo:hi]

    def _shard_grads(self, p):
        return self.grad_layout == "shard" and self._is_sharded_shape(p)

    def _grad_accumulator_bytes(self):
        if self.grad_layout != "shard":
            return super()._grad_accumulator_bytes()
        return sum(p.numel() * 2 // (self._world_size if self._is_sharded_shape(p) else 1)
                   for p in self._offload_params)

    def _state_shape(self, p, key):
        if key == "grad":
            full = super()._state_shape(p, key)
            if full == p.shape and self._shard_grads(p):
                return (p.shape[0] // self._world_size, *p.shape[1:])
            return full
        if self._is_sharded_shape(p):
            return (p.shape[0] // self._world_size, *p.shape[1:])
        return p.shape

    def _seed_master(self, p, master):
        src = p.data
        if p in self._quant_params:
            full = torch.empty(p.shape, dtype=torch.float32, device="cpu")
            full.copy_(src)  # dequantizes
            src = full
        if self._is_sharded_shape(p):
            lo, hi = self._rows(p)
            src = src[lo:hi]
        master.copy_(src)

    def _alloc_pinned_states(self, params, numa_node):
        for p in params:
            if self._is_sharded_shape(p):
                self._sharded.add(p)
        super()._alloc_pinned_states(params, numa_node)

    def _log_prefix(self):
        return f"[rank {self._rank}] "

    def _resolve_seed(self, seed):
        if seed is not None or self._world_size <= 1:
            return super()._resolve_seed(seed)
        box = [super()._resolve_seed(None) if self._rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self._pg, 0), group=self._pg)
        return box[0]

    def _copy_master(self, p, tensor):
        self._engine.invalidate_prefetched()  # a copy loaded ahead of time would be stale
        if p in self._sharded:
            lo, hi = self._rows(p)
            tensor = tensor[lo:hi]
        self.state[p]["master_params"].copy_(tensor)

    # ------------------------------------------------------------ comm set-up
    def _setup_comm(self, model):
        want = self._requested_comm
        if self._world_size <= 1 or not self._cuda:
            if want == "symm" and self._world_size > 1:
                raise RuntimeError("comm='symm' needs CUDA devices")
            return
        if want == "nccl":
            return
        if self.grad_residency != "device":
            if want == "symm":
                raise RuntimeError("comm='symm' needs grad_residency='device'")
            return
        from . import symm

        try:
            self._symm = symm.SymmZero1(self, model, timeout_ms=self._wait_timeout_ms)
            self.comm = "symm"
            self._fused_quant = {}  # payload addresses changed: plans are rebuilt on first use
        except Exception as e:
            if want == "symm":
                raise
            import warnings

            warnings.warn(f"DistributedOffloadAdam: symmetric-memory path unavailable ({e}); "
                          f"using torch.distributed collectives")

    # ------------------------------------------------------- collective helpers
    def _avg_all_reduce(self, t):
        """In-place average over ranks (fp32 accumulate for bf16 on CPU/gloo)."""
        if self._world_size <= 1:
            return
        if t.is_cuda:
            dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self._pg)
        else:
            f = t.float()
            dist.all_reduce(f, op=dist.ReduceOp.SUM, group=self._pg)
            t.copy_((f / self._world_size).to(t.dtype))

    def _avg_reduce_scatter(self, full, p):
        """Average over ranks of ``full`` restricted to this rank's rows."""
        lo, hi = self._rows(p)
        if full.is_cuda:
            out = torch.empty((hi - lo, *p.shape[1:]), dtype=full.dtype, device=full.device)
            dist.reduce_scatter_tensor(out.view(-1), full.contiguous().view(-1),
                                       op=dist.ReduceOp.AVG, group=self._pg)
            return out
        f = full.float()
        dist.all_reduce(f, op=dist.ReduceOp.SUM, group=self._pg)
        return (f[lo:hi] / self._world_size).to(full.dtype).contiguous()

    def _all_gather_rows(self, dst_full, local_rows):
        if dst_full.is_cuda:
            dist.all_gather_into_tensor(dst_full.view(-1), local_rows.contiguous().view(-1), group=self._pg)
        else:
            parts = [torch.empty_like(local_rows) for _ in range(self._world_size)]
            dist.all_gather(parts, local_rows.contiguous(), group=self._pg)
            dst_full.copy_(torch.cat(parts, dim=0).view_as(dst_full))

    def _side(self):
        """Context that routes torch ops (and collectives) to the optimizer stream."""
        if self._cuda:
            return torch.cuda.stream(self._engine.opt_stream)
        import contextlib

        return contextlib.nullcontext()

    # ------------------------------------------------------------------- hooks
    @torch.no_grad()
    def _inplace_grad_hook(self, p):
        if p.grad is None:
            return
        if not self.ready_for_optimizer_step or self._world_size <= 1:
            return super()._inplace_grad_hook(p)
        grad = self._take_grad(p)
        st = self.state[p]
        grad_ops.grad_accumulate(st["grad"], st["grad"], grad, scratch=self._scratch_main)
        if self._symm is None:  # the symmetric path averages all small tensors in one bucket later
            self._avg_all_reduce(st["grad"])
            if self._want_norm():
                grad_ops.grad_accumulate(None, st["grad"], None, sumsq=self._slot(p),
                                         scratch=self._scratch_main)
        if self._step_in_backward:
            st["step"] += 1
            self._pending_inplace.append(p)

    @torch.no_grad()
    def _grad_hook(self, p):
        if p.grad is None:
            return
        symm = self._symm is not None and self._symm.handles(p)
        if self._world_size > 1 and self._shard_grads(p):
            self._pace_prefetch(1)
            if symm:
                return self._symm.grad_hook_window(p, self.ready_for_optimizer_step)
            return self._shard_grad_hook(p, self.ready_for_optimizer_step)
        if not self.ready_for_optimizer_step or self._world_size <= 1:
            if symm:
                self._pace_prefetch(1)
                return self._symm.accumulate(p, self._take_grad(p))
            return super()._grad_hook(p)
        self._pace_prefetch(1)
        if symm:
            return self._symm.grad_hook_last(p)
        # ---- last micro-batch, torch.distributed collectives
        grad = self._take_grad(p)
        st = self.state[p]
        eng = self._engine
        eng.fork_from_main()
        with self._side():
            acc = self._dev_grad.pop(p, None)
            if acc is not None:
                grad_ops.grad_accumulate(acc, acc, grad, scratch=eng.scratch, use_cuda=self._cuda,
                                         stream=self._opt_stream_handle())
                full = acc
            elif st["host_grad_valid"]:
                # the kernel reads the pinned buffer directly: the copy of the previous
                # micro-batch into it (D2H stream) has to be complete
                eng.wait_host_grad(self._pid[p])
                grad_ops.grad_accumulate(grad, grad, st["grad"], use_cuda=self._cuda,
                                         stream=self._opt_stream_handle())
                full = grad
                st["host_grad_valid"] = False
            else:
                full = grad
            if p in self._sharded:
                red = self._avg_reduce_scatter(full, p)
            else:
                self._avg_all_reduce(full)
                red = full
            if self.max_grad_norm is not None:
                grad_ops.grad_accumulate(None, red, None, sumsq=self._slot(p), scratch=eng.scratch,
                                         use_cuda=self._cuda, stream=self._opt_stream_handle())
        eng._retain(grad)
        if acc is not None:
            eng._retain(acc)
        self._dev_grad[p] = red  # reduced gradient (slice for sharded) waits for its step
        if self._step_in_backward:
            self._step_offload(p, self._param2group[p])

    def _shard_grad_hook(self, p, last):
        """``grad_layout='shard'``: average this micro-batch's gradient over the ranks
        now and accumulate only this rank's rows."""
        grad = self._take_grad(p)
        st = self.state[p]
        eng = self._engine
        s = self._opt_stream_handle()
        eng.fork_from_main()
        with self._side():
            red = self._avg_reduce_scatter(grad, p)
            total = None
            if self.grad_residency == "device":
                acc = self._dev_grad.get(p)
                if acc is None:
                    total = red
                else:
                    grad_ops.grad_accumulate(acc, acc, red, scratch=eng.scratch, use_cuda=self._cuda, stream=s)
                    total = acc
                self._dev_grad[p] = total
            elif last:
                if st["host_grad_valid"]:
                    eng.wait_host_grad(self._pid[p])  # as above: a zero-copy read of the pinned buffer
                    grad_ops.grad_accumulate(red, red, st["grad"], use_cuda=self._cuda, stream=s)
                    st["host_grad_valid"] = False
                total = red
                self._dev_grad[p] = total
            if last and self.max_grad_norm is not None:
                grad_ops.grad_accumulate(None, total, None, sumsq=self._slot(p), scratch=eng.scratch,
                                         use_cuda=self._cuda, stream=s)
        if self.grad_residency != "device" and not last:
            eng.grad_to_host(self._pid[p], st["grad"], red, first=not st["host_grad_valid"])
            st["host_grad_valid"] = True
        eng._retain(grad)
        eng._retain(red)
        if last and self._step_in_backward:
            self._step_offload(p, self._param2group[p])

    def _opt_stream_handle(self):
        return self._engine.opt_stream.cuda_stream if self._cuda else 0

    # ------------------------------------------------------------- step pieces
    def _param_view(self, p):
        return self._shard_slice(p) if p in self._sharded else p.data

    def _step_extra(self, p):
        if self._symm is not None and self._symm.handles(p):
            return self._symm.step_extra(p)
        return {}

    def _after_param_update(self, p):
        if self._symm is not None and self._symm.handles(p):
            return self._symm.after_param_update(p)
        if p not in self._sharded:
            return
        if p in self._quant_params:
            return  # handled in _step_quant
        with self._side():
            self._all_gather_rows(p.data, self._shard_slice(p))

    def _fused_quant_ok(self, p):
        """True when the fused Adam + re-quantize + push kernels take this weight."""
        eng = self._engine
        C = getattr(eng, "C", None)
        return bool(self._cuda and eng._native is not None and p.KERNEL_FORMAT and p.dim() == 2
                    and p.kernel_scale_dtype() in (torch.float32, torch.bfloat16, torch.float16)
                    and C.adam_quant_supported(p.KERNEL_FORMAT, p.shape[1], p.kernel_group()))

    def _quant_replicas(self, p):
        if self._symm is not None and self._symm.handles(p):
            return self._symm.quant_replicas(p)
        return super()._quant_replicas(p)

    def _quant_amax_is_global(self, p):
        return self._symm is not None and self._symm.handles(p) and p in self._sharded

    def _combine_amax(self, p, plan):
        if self._quant_amax_is_global(p):
            self._symm.combine_amax(plan["local_amax"], plan["tensor_amax"])

    def _fused_quant_plan(self, p):
        if p in self._sharded and not (self._symm is not None and self._symm.handles(p)):
            return None  # rows divided among ranks, no peer mappings: the collective route below
        return super()._fused_quant_plan(p)

    def _grad_is_persistent(self, p):
        # the reduced slices of the clip path and the shard accumulators are buffers of the
        # symmetric-memory path, alive as long as the optimizer
        return self._symm is not None and self._symm.handles(p) and p in self._symm.red

    def _step_quant(self, p, group, st, dev_grad, host_grad, clip_coef, fork=True):
        if p not in self._sharded or self._fused_quant_plan(p) is not None:
            return super()._step_quant(p, group, st, dev_grad, host_grad, clip_coef, fork=fork)
        # sharded quantized parameter over torch.distributed: the owner of each row range
        # updates its master slice, quantizes those rows and the PACKED rows are gathered
        # (at most one byte per element on the wire instead of four, and no replica
        # re-quantizes rows it does not own).  The reference gathers the fp32 master and
        # re-quantizes the whole weight on every rank
        # (src/offload_adam/distributed_offload_adam.py:250-262).
        eng = self._engine
        from ..ops.adam_step import adam_step

        q = p.data
        lo, hi = self._rows(p)
        if self._cuda:
            eng.fork_from_main()
        with self._side():
            master = st["master_params"].to(self.device, non_blocking=True) if self._cuda \
                else st["master_params"]
            states = {"grad": dev_grad, "exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"],
                      "master_params": master}
            amax = torch.zeros(1, dtype=torch.float32, device=master.device) if q.USES_TENSOR_AMAX else None
            adam_step(self.mode, None, states, *self._hp(group), st["step"],
                      decoupled_weight_decay=self.decoupled_weight_decay, clip_coef=clip_coef, amax=amax,
                      max_ctas=eng.max_ctas, stream=self._opt_stream_handle(), use_cuda=self._cuda)
            if amax is not None:
                dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self._pg)
            shard, views = q.row_shard(lo, hi)
            shard._quantize_into(master, amax)
            for full, view, part in zip(q._payload(), views, shard._payload()):
                if view.shape == full.shape:
                    continue  # per-tensor quantity: every rank wrote the same value
                self._gather_payload(full, view, part)
            if self._cuda:
                st["master_params"].copy_(master, non_blocking=True)
        eng._retain(dev_grad)

    def _gather_payload(self, full, view, part):
        """All-gather one packed payload tensor from per-rank row ranges."""
        if part.data_ptr() == view.data_ptr():
            # row-major payload: ranks own consecutive byte ranges of ``full``; in place
            flat = full.view(-1)
            mine = part.view(-1)
            if flat.element_size() == 1:
                flat, mine = flat.view(torch.uint8), mine.view(torch.uint8)
            if full.is_cuda:
                dist.all_gather_into_tensor(flat, mine, group=self._pg)
            else:
                parts = [torch.empty_like(mine) for _ in range(self._world_size)]
                dist.all_gather(parts, mine.clone(), group=self._pg)
                flat.copy_(torch.cat(parts))
            return
        # transposed payload (rows of the weight are columns here): gather the
        # contiguous temporaries and lay them side by side
        dim = next(d for d in range(full.dim()) if view.shape[d] != full.shape[d])
        parts = [torch.empty_like(part) for _ in range(self._world_size)]
        dist.all_gather(parts, part, group=self._pg)
        torch.cat(parts, dim=dim, out=full)

    def _global_clip_coef(self):
        if self.max_grad_norm is None:
            return None
        if self._world_size <= 1:
            return super()._global_clip_coef()
        if self._symm is not None:
            return self._symm.global_clip_coef()
        # sharded params contribute disjoint slices on every rank; replicated ones are
        # identical everywhere and are counted by rank 0 only
        self._engine.join_main(wait_writeback=False)
        idx = [self._pid[p] for p in self._all_params if p in self._sharded or self._rank == 0]
        index = torch.tensor(idx, dtype=torch.int32, device=self.device)
        local = torch.zeros(1, dtype=torch.float32, device=self.device)
        grad_ops.clip_finalize(self._normsq, index, None, self.max_grad_norm, total_sq=local)
        dist.all_reduce(local, op=dist.ReduceOp.SUM, group=self._pg)
        grad_ops.clip_finalize(None, None, local, self.max_grad_norm, coef_norm=self._clip)
        return self._clip[0:1]

    def _finish_step(self):
        if self._symm is None:
            return super()._finish_step()
        stepped = self._step_dirty or bool(self._pending_inplace)
        self._symm.before_finish()
        super()._finish_step()
        if stepped:
            self._symm.after_finish()

    def synchronize(self):
        super().synchronize()
        if self._symm is not None:
            self._symm.check_status(blocking=True)

    # ------------------------------------------------- checkpoints across world sizes
    def _gather_rows_to(self, shard, dst):
        """Rows of all ranks stacked in rank order, on rank ``dst`` (None elsewhere)."""
        world = self._world_size
        if world <= 1:
            return shard.detach().clone()
        if dist.get_backend(self._pg) == "gloo" or not self._cuda:
            parts = [torch.empty_like(shard, device="cpu") for _ in range(world)] if self._rank == dst else None
            dist.gather(shard.detach().cpu().contiguous(), parts, dst=dist.get_global_rank(self._pg, dst),
                        group=self._pg)
            return torch.cat(parts, dim=0) if self._rank == dst else None
        dev = shard.detach().to(self.device).contiguous()
        full = torch.empty((world * dev.shape[0], *dev.shape[1:]), dtype=dev.dtype, device=self.device)
        dist.all_gather_into_tensor(full.view(-1), dev.view(-1), group=self._pg)
        return full.cpu() if self._rank == dst else None

    @torch.no_grad()
    def consolidated_state_dict(self, dst=0):
        """``state_dict()`` with every sharded state tensor replaced by the full-shape
        tensor (the rows of all ranks), returned on rank ``dst`` of the group and ``None``
        elsewhere.  Collective: every rank must call it.  The result loads into an
        optimizer of any world size (``load_offload_state_dict`` slices full-shape tensors
        to the caller's rows) and into a single-GPU ``OffloadAdam``.  The reference has no
        checkpoint logic across ranks."""
        self.synchronize()
        sd = super().state_dict()
        ids = [i for g in sd["param_groups"] for i in g["params"]]
        live = [p for g in self.param_groups for p in g["params"]]
        out_state = {}
        for idx, p in zip(ids, live):
            src = sd["state"].get(idx)
            if src is None:
                continue
            entry = {}
            for k, v in src.items():
                if isinstance(v, torch.Tensor) and k == "grad":
                    continue  # transient accumulator, never part of a resume
                if isinstance(v, torch.Tensor) and p in self._sharded and k in self._non_grad_keys:
                    v = self._gather_rows_to(v, dst)
                elif isinstance(v, torch.Tensor):
                    v = v.detach().cpu().clone()
                entry[k] = v
            out_state[idx] = entry
        if self._rank != dst:
            return None
        return {"state": out_state, "param_groups": sd["param_groups"]}

    @torch.no_grad()
    def load_offload_state_dict(self, state_dict):
        """As in :class:`OffloadAdam`; state tensors of sharded parameters may also come
        in full shape (``consolidated_state_dict()`` output, or the ``state_dict()`` of a
        single-GPU optimizer): this rank's rows are taken."""
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        live = [p for g in self.param_groups for p in g["params"]]
        if len(ids) == len(live):
            state = dict(state_dict["state"])
            for idx, p in zip(ids, live):
                src = state.get(idx)
                if src is None or p not in self._sharded:
                    continue
                lo, hi = self._rows(p)
                sliced = {}
                for k, v in src.items():
                    if (isinstance(v, torch.Tensor) and k in self._non_grad_keys
                            and tuple(v.shape) == tuple(p.shape) and hi - lo != p.shape[0]):
                        v = v[lo:hi]
                    sliced[k] = v
                state[idx] = sliced
            state_dict = {"state": state, "param_groups": state_dict["param_groups"]}
        return super().load_offload_state_dict(state_dict)
