"""``OffloadAdam``: Adam/AdamW whose optimizer state lives in pinned host memory.

Public contract (constructor arguments, the ``ready_for_optimizer_step`` flag,
``step`` / ``zero_grad`` / ``state_dict`` / ``load_master_*`` and the per
parameter state layout) follows the reference optimizer
(reference: src/offload_adam/offload_adam.py:39-678).  Two execution paths are
selected by ``max_grad_norm``:

* ``None``: the step of each parameter is enqueued from its
  post-accumulate-grad hook on the last micro-batch and overlaps the rest of
  backward; ``step()`` only joins the side streams.
* a float: backward accumulates gradients and per-parameter squared norms;
  ``step()`` turns them into one clip coefficient (a device scalar, no host
  sync) and streams every parameter through the clip-fused step kernel.

How this implementation differs underneath:

* state tensors are views into a few NUMA-bound pinned segments
  (``utils.pinned_alloc.PinnedArena``) instead of one registration per tensor;
* the transfer layer (``engine.TransferEngine``) either lets the step kernel
  read/write host memory directly over PCIe (``transfer='zero_copy'``) or
  pipelines chunks through a circular staging buffer in device memory
  (``transfer='staged'``), which also takes in the next step's state while
  forward/backward run and lets the last step's write-backs drain behind the next
  forward pass; there is no host synchronisation;
* gradient accumulation across micro-batches can stay in HBM
  (``grad_residency='device'``; ``'auto'`` picks it when the accumulators fit a
  budget) or live on the host as in the reference (``'host'``), in which case a
  single read-modify-write kernel per micro-batch replaces the D2H + H2D +
  ``add_`` round trip;
* all small parameters are stepped by one multi-tensor launch.
"""

from __future__ import annotations

import os
import random
import time
import warnings

import torch
from torch.optim.optimizer import Optimizer

from ._master import MasterLoadingMixin, is_quant
from .engine import TransferEngine
from .ops import grad_ops
from .ops.adam_step import STEP_FNS, adam_step
from .utils.pinned_alloc import PinnedArena, numa_node_free_bytes, resolve_numa_target

_BF16 = torch.bfloat16


def get_leaf_modules_with_params(module):
    """Modules that directly own a trainable parameter, in registration (= forward
    definition) order.  The reference walks the children and keeps the leaves
    (reference: src/offload_adam/offload_adam.py:26-36), which silently leaves out
    parameters held by a module that also has children, and every parameter of a model
    that is itself a leaf; both are included here."""
    return [m for m in module.modules()
            if any(p.requires_grad for p in m.parameters(recurse=False))]


def _offload_layout(extra_name=None, extra_dtype=None):
    d = {"grad": _BF16, "exp_avg": _BF16, "exp_avg_sq": _BF16}
    if extra_name:
        d[extra_name] = extra_dtype
    return d


class OffloadAdam(MasterLoadingMixin, Optimizer):
    """Adam optimizer that keeps gradients and optimizer state in host memory.

    Args:
        model (nn.Module): the module whose trainable parameters are optimized
            (pass the module, not its parameters: hooks are installed on it).
        lr, betas, eps, weight_decay: Adam hyper-parameters.
        mode: ``'stochastic_rounding'`` (default), ``'fp32_master'``,
            ``'fp31_master'`` or ``'fp32_master_custom_rounding'``.
        max_grad_norm: L2 global-norm clipping threshold, or None to run the step
            inside backward.
        numa_node: ``'auto'`` binds pinned memory to the GPU's NUMA node, an int
            picks a node, None disables binding.
        decoupled_weight_decay: AdamW-style decay.
        inplace_param_threshold: parameters with fewer elements keep state and
            gradient on the GPU (default 1 Mi elements; 0 offloads everything).
        prefetch_policy: ``'eager'`` or ``'lazy'``.  In the reference the policy decides
            which owner module of a shared (tied) parameter brings its state to the GPU
            ahead of the step, and how long that state stays there.  Here state is
            streamed through a staging buffer in the order of the steps, so the policy
            only decides where a shared parameter sits in the early-load order of the
            step-in-backward path before that order has been observed: ``'eager'`` places
            it where its last owner module sits (the first one backward reaches),
            ``'lazy'`` where its first owner sits (the input side, reached last).  From
            the second step on the observed order is used under both policies, and the
            clipping path always steps in parameter order.
        verbose: non-zero prints allocation summaries.
        transfer: ``'auto'`` | ``'zero_copy'`` | ``'staged'`` (see module doc).
        grad_residency: ``'auto'`` | ``'host'`` | ``'device'``.
        device_grad_budget: bytes of HBM ``'auto'`` may spend on gradient
            accumulators (default: a quarter of the device's memory).
        prefetch_pacing: who issues the early H2D.  ``'thread'`` (default): a helper
            thread of the copy engine, which keeps ``prefetch_inflight`` copies outstanding
            whatever the training loop is doing; ``'hooks'``: the training thread itself,
            one chunk at every forward pre-hook of a leaf module and every gradient hook.
        prefetch_inflight: early-H2D chunks allowed in the copy engine at once (default 2:
            a copy the caller issues, such as an input batch, waits behind two chunks at
            most, a few milliseconds); 0 queues everything that fits in the staging buffer as soon as a step
            ends, which keeps the link busy through the step but makes other H2D copies
            wait behind it.
        debug_serialize: debugging aid against stream races.  Every transfer and step
            finishes before the call that enqueued it returns; no helper threads, no early
            loads.  Results must equal the overlapped run bit for bit; a difference points
            at a missing dependency between streams.
        debug_canaries: debugging aid against kernels that write past their operands
            (staged transfer).  Every chunk in the staging buffer and every resident tensor is
            followed by 256 bytes of a known pattern that a small kernel verifies after the
            chunk's step; ``synchronize()`` raises, naming the tensor, when a guard was
            overwritten.
        nvtx: wrap ``step()``, the gradient hooks and the clip reduction in NVTX ranges
            (``oab.*``) for timeline profilers.
        async_writeback: issue the D2H write-backs of the staged transfer from a helper
            thread, so that the caller never blocks on a full stream queue (default).
        chunk_elems: elements per staged chunk (default 8 Mi).
        ring_slots: smallest number of full-width chunks the staging buffer must hold,
            whatever ``staging_bytes`` says (default 4).
        staging_bytes: HBM set aside for the circular staging buffer of the staged
            transfer.  State of the first tensors of the next step is brought into it
            while forward/backward run and the last write-backs of a step drain from it
            while the next forward runs, so the host link works through the whole
            iteration instead of only during the exposed part of the step.  ``None``
            (default): this rank's state size, at most a quarter of the device's memory
            and a third of the memory that is free when the optimizer is built.  A few hundred MB are
            enough for the step itself; everything above that buys overlap.
        keep_resident: let state that fits in the staging buffer stay there between
            steps (default).  Such tensors are loaded once, stepped with one launch and
            written back to the host after every step, so the host copy stays current and
            authoritative while nothing crosses the host link towards the GPU for them.
            When the buffer cannot hold everything, the tensors that are stepped last
            stay and the others stream through the rest of the buffer.  ``False``
            streams everything every step.
        resident_writeback: ``'step'`` (default) copies resident state back to the host after
            every step.  ``'on_demand'`` copies it back only when the host copy is asked for
            (``state_dict()``, ``synchronize()``, ``wait_writeback()``, ``close()``): between
            those calls the resident tensors' host buffers are stale and nothing of them
            crosses the host link in either direction, like the small tensors that
            ``inplace_param_threshold`` keeps on the GPU.
        max_ctas: grid cap of the streaming kernels (0: kernel default); small
            values leave the SMs to the concurrent backward GEMMs.
        seed: seeds the stochastic-rounding stream.
    """

    supported_modes = {
        "stochastic_rounding": {"step": STEP_FNS["stochastic_rounding"], "offload": _offload_layout()},
        "fp32_master": {
            "step": STEP_FNS["fp32_master"],
            "offload": _offload_layout("master_params", torch.float32),
        },
        "fp31_master": {
            "step": STEP_FNS["fp31_master"],
            "offload": _offload_layout("rounding_error", torch.int16),
        },
        "fp32_master_custom_rounding": {
            "step": STEP_FNS["fp32_master_custom_rounding"],
            "offload": _offload_layout("rounding_error", torch.int16),
        },
    }

    _DEFAULT_INPLACE_PARAM_THRESHOLD = 1024 * 1024

    def __init__(self, model, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 mode="stochastic_rounding", max_grad_norm=None, numa_node="auto",
                 decoupled_weight_decay=False, inplace_param_threshold=None,
                 prefetch_policy="eager", verbose=0, *, transfer="auto", grad_residency="auto",
                 device_grad_budget=None, chunk_elems=None, ring_slots=4, max_ctas=0,
                 max_inflight_bytes=8 << 30, staging_bytes=None, prefetch_inflight=2, prefetch_pacing="thread", async_writeback=True,
                 debug_serialize=False, nvtx=False, seed=None, keep_resident=True, debug_canaries=False,
                 resident_writeback="step"):
        if prefetch_policy not in ("eager", "lazy"):
            raise ValueError(f"prefetch_policy must be 'eager' or 'lazy' (got {prefetch_policy!r})")
        if grad_residency not in ("auto", "host", "device"):
            raise ValueError(f"grad_residency must be 'auto', 'host' or 'device' (got {grad_residency!r})")
        assert mode in self.supported_modes, (
            f"Invalid mode: {mode}, available modes: {list(self.supported_modes)}"
        )
        self._prefetch_policy = prefetch_policy
        self.mode = mode
        self.step_fn = self.supported_modes[mode]["step"]
        self.offload_config = self.supported_modes[mode]["offload"]
        self.offload_state_keys = list(self.offload_config)
        self._non_grad_keys = [k for k in self.offload_state_keys if k != "grad"]
        self._has_master = "master_params" in self.offload_config
        self.max_grad_norm = max_grad_norm
        self._step_in_backward = max_grad_norm is None
        self.decoupled_weight_decay = decoupled_weight_decay
        self.verbose = verbose
        self.ready_for_optimizer_step = False
        self._rng = random.Random(self._resolve_seed(seed))
        self.keep_resident = bool(keep_resident)

        # ---- collect parameters: unique by identity, count owning leaf modules
        modules = get_leaf_modules_with_params(model)
        params, owners = [], {}
        for m in modules:
            for p in m.parameters(recurse=False):
                if not p.requires_grad:
                    continue
                if id(p) not in owners:
                    owners[id(p)] = 0
                    params.append(p)
                owners[id(p)] += 1
        shared = [p for p in params if owners[id(p)] > 1]
        if shared and prefetch_policy == "eager":
            warnings.warn(
                f"OffloadAdam: {len(shared)} parameter(s) shared across multiple leaf modules "
                f"({sum(p.numel() for p in shared):,} elements; e.g. tied embeddings). With "
                f"prefetch_policy='eager' early work for them is triggered by the first owner "
                f"module reached in backward. Pass prefetch_policy='lazy' to defer it to the "
                f"input-side module.",
                stacklevel=2,
            )
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

        self._quant_params = {p for p in params if is_quant(p)}
        if self._quant_params and mode != "fp32_master":
            raise ValueError(
                f"QAT params require mode='fp32_master'; got {mode!r} "
                f"({len(self._quant_params)} quant params detected)"
            )
        self._quant_master_warned = False

        if inplace_param_threshold is None:
            inplace_param_threshold = self._DEFAULT_INPLACE_PARAM_THRESHOLD
        self.inplace_param_threshold = inplace_param_threshold
        self._inplace_params = {
            p for p in params if p.numel() < inplace_param_threshold and p not in self._quant_params
        }
        self._offload_params = [p for p in params if p not in self._inplace_params]
        self._all_params = params
        self._pid = {p: i for i, p in enumerate(params)}
        self._param2group = {p: g for g in self.param_groups for p in g["params"]}
        self.device = params[0].device if params else torch.device("cpu")
        self._cuda = self.device.type == "cuda"
        elsewhere = {str(p.device) for p in params if p.device != self.device}
        if elsewhere:
            raise ValueError(
                f"{type(self).__name__} drives one device: parameters live on {self.device} and also on "
                f"{sorted(elsewhere)}; use one process per GPU (DistributedOffloadAdam) instead")
        not_bf16 = {str(p.dtype) for p in params if p.dtype != _BF16 and p not in self._quant_params}
        if not_bf16:
            raise ValueError(f"{type(self).__name__} expects bfloat16 parameters (found {sorted(not_bf16)}); "
                             "call model.to(torch.bfloat16) first")

        # position (in forward order) of the owner module that stands for a parameter in
        # the first guess of the backward order: the first owner under 'lazy', the last
        # under 'eager' (they differ for shared parameters only)
        self._owner_pos = {}
        for pos, m in enumerate(modules):
            for p in m.parameters(recurse=False):
                if p.requires_grad and p not in self._inplace_params:
                    if prefetch_policy == "lazy":
                        self._owner_pos.setdefault(p, pos)
                    else:
                        self._owner_pos[p] = pos

        # ---- where gradient accumulators live
        grad_bytes = self._grad_accumulator_bytes()
        if grad_residency == "auto":
            if self._cuda:
                if device_grad_budget is None:
                    device_grad_budget = torch.cuda.get_device_properties(self.device).total_memory // 4
                grad_residency = "device" if grad_bytes <= device_grad_budget else "host"
            else:
                grad_residency = "host"
        self.grad_residency = grad_residency
        if chunk_elems is None:
            # large chunks: every chunk costs five operations on the D2H stream and a
            # stream takes about a thousand pending operations before enqueueing blocks
            chunk_elems = 8 << 20
        self._nvtx = bool(nvtx) and self._cuda
        self._owner_pid = os.getpid()
        self.prefetch_inflight = int(prefetch_inflight)
        if prefetch_pacing not in ("thread", "hooks"):
            raise ValueError(f"prefetch_pacing must be 'thread' or 'hooks', got {prefetch_pacing!r}")
        if resident_writeback not in ("step", "on_demand"):
            raise ValueError(f"resident_writeback must be 'step' or 'on_demand', got {resident_writeback!r}")
        self.resident_writeback = resident_writeback
        self.prefetch_pacing = prefetch_pacing
        self._engine = TransferEngine(
            self.device, mode, len(params), transfer=transfer, chunk_elems=chunk_elems,
            ring_slots=ring_slots, max_ctas=max_ctas, max_inflight_bytes=max_inflight_bytes,
            staging_bytes=self._resolve_staging_bytes(staging_bytes),
            async_writeback=async_writeback, serialize=debug_serialize, canaries=debug_canaries,
            lazy_resident=resident_writeback == "on_demand",
        )
        self.transfer = self._engine.transfer
        self.h2d_stream = self._engine.h2d_stream
        self.d2h_stream = self._engine.d2h_stream
        self.opt_stream = self._engine.opt_stream

        self._dev_grad = {}       # param -> accumulated gradient tensor on the device
        self._pending_inplace = []  # small params whose step is due at the next join
        self._normsq = torch.zeros(max(1, len(params)), dtype=torch.float32, device=self.device)
        self._norms = torch.zeros_like(self._normsq)
        self._clip = torch.ones(2, dtype=torch.float32, device=self.device)
        self._multi = None
        self._step_dirty = False
        self._hook_order_prev, self._hook_order_cur = None, []
        self._pf_order, self._pf_idx, self._pf_off = None, 0, 0
        # main-stream reductions get their own scratch: the engine's belongs to its side stream
        self._scratch_main = grad_ops.sumsq_scratch(self.device)

        self._fused_quant = {}   # quantized param -> dict(chunk, spec) or None (unfused route)
        self._master_tmp = None  # device copy of an updated NVFP4 master between its two passes
        self._amax = None
        self._register_hooks(model, modules, params)
        self._numa_precheck(self._offload_params, numa_node)
        self._alloc_pinned_states(self._offload_params, numa_node)
        self._alloc_inplace_states(self._inplace_params)
        self._choose_resident()
        self._constructed = True

    def _resolve_seed(self, seed):
        """Seed of the stochastic-rounding stream.  ``None`` draws from Python's global
        ``random`` module, so that ``random.seed(...)`` makes runs repeatable as it does
        for the reference (reference: src/offload_adam/kernels/stochastic_rounding.py:98-99)."""
        return random.getrandbits(63) if seed is None else seed

    # ------------------------------------------------------- resident state
    def _step_order_guess(self):
        """Offloaded parameters in the order their steps are expected: parameter order
        on the clipping path; on the step-in-backward path the order observed in the
        previous step or, before there is one, owner modules from the output side
        back to the input side."""
        if not self._step_in_backward:
            return [p for g in self.param_groups for p in g["params"] if p not in self._inplace_params]
        if self._hook_order_prev:
            return list(self._hook_order_prev)
        pos = self._owner_pos
        return sorted((p for p in self._offload_params), key=lambda p: -pos.get(p, 0))

    def _state_elems(self, p):
        return self.state[p]["exp_avg"].numel()

    def _choose_resident(self):
        """Pick the tensors whose state stays in the staging buffer (see ``keep_resident``).
        The tail of the step order is taken: the streamed tensors then go first, their
        write-backs are not queued behind gigabytes of resident state, and the chunks they
        occupy are free again when the next loads want them."""
        eng = self._engine
        self._resident = set()
        if not (self.keep_resident and self._cuda and eng.can_make_resident and self.grad_residency == "device"):
            return
        per_elem = sum(torch.empty(0, dtype=self.offload_config[k]).element_size() for k in self._non_grad_keys)
        need = {p: self._state_elems(p) * per_elem + 768 for p in self._offload_params}
        total = sum(need.values())
        budget = eng.resident_budget(total)
        for p in reversed(self._step_order_guess()):
            if need[p] > budget:
                break
            if not eng.make_resident(self._pid[p], self._state_elems(p)):
                break
            budget -= need[p]
            self._resident.add(p)
        if self.verbose > 0 and self._resident:
            print(f"{self._log_prefix()}state resident in the staging buffer: {len(self._resident)} of "
                  f"{len(self._offload_params)} tensors, {eng.resident_bytes / 2**30:.2f} GiB")

    def add_param_group(self, param_group):
        if getattr(self, "_constructed", False):
            raise NotImplementedError(
                f"{type(self).__name__} partitions, hooks and allocates pinned state for its "
                "parameters at construction; build a new optimizer for a changed parameter set "
                "(close() this one first)")
        return super().add_param_group(param_group)

    # ------------------------------------------------------------------ setup
    def _register_hooks(self, model, modules, params):
        # No module-level backward pre-hooks: the streaming transfer modes have nothing
        # to park on the GPU ahead of a parameter's gradient, and full backward hooks
        # would add an autograd node per leaf-module call.
        self._hook_handles = []
        for i, p in enumerate(params):
            st = self.state[p]
            st["step"] = 0
            if self.max_grad_norm is not None:
                st["grad_norm"] = self._norms[i]
            if p in self._inplace_params:
                self._hook_handles.append(p.register_post_accumulate_grad_hook(self._inplace_grad_hook))
            else:
                self._hook_handles.append(p.register_post_accumulate_grad_hook(self._grad_hook))
                st["host_grad_valid"] = False
        # the next forward must see every update even if the caller skipped step(); so must
        # a state_dict() of the model taken right after backward (steps of the small
        # parameters are deferred to this point on the step-in-backward path)
        self._hook_handles.append(model.register_forward_pre_hook(lambda *_: self._on_forward()))
        if hasattr(model, "register_state_dict_pre_hook"):
            self._hook_handles.append(model.register_state_dict_pre_hook(lambda *_: self._finish_step()))
        # pacing points for the early H2D during forward (plain forward hooks add no
        # autograd nodes); not needed when the helper thread paces
        for m in (modules if self.prefetch_pacing == "hooks" else ()):
            if any(p.requires_grad and p not in self._inplace_params for p in m.parameters(recurse=False)):
                self._hook_handles.append(m.register_forward_pre_hook(lambda *_: self._pace_prefetch(1)))

    def _grad_accumulator_bytes(self):
        """Bytes of the bf16 gradient accumulators of the offloaded parameters."""
        return sum(p.numel() * 2 for p in self._offload_params)

    def _state_shape(self, p, key):
        """Shape of one host state tensor (subclasses shard the non-grad ones).  With
        device-resident accumulators no host gradient buffer is needed: the ``grad``
        entry stays in the state dict as an empty placeholder."""
        if key == "grad" and self.grad_residency == "device":
            return (0,)
        return p.shape

    def _estimate_pinned_bytes(self, params):
        total = 0
        for p in params:
            for key, dtype in self.offload_config.items():
                n = 1
                for d in self._state_shape(p, key):
                    n *= d
                total += n * torch.empty(0, dtype=dtype).element_size()
        return total

    def _numa_precheck(self, params, numa_node):
        """Warn when the bound node cannot hold this rank's share of pinned state
        (soft binding then spills to remote nodes at some H2D cost)."""
        target = resolve_numa_target(numa_node, self.device if self._cuda else None) if self._cuda else None
        if target is None or not params:
            return
        free = numa_node_free_bytes(target)
        if free is None:
            return
        need = self._estimate_pinned_bytes(params)
        world = getattr(self, "_world_size", 1)
        share = free // max(1, world)
        if need > share:
            gib = 1024**3
            warnings.warn(
                f"OffloadAdam: need {need / gib:.1f} GB pinned on NUMA node {target} "
                f"({world} rank(s) sharing) but fair share is {share / gib:.1f} GB; "
                f"~{(need - share) / gib:.1f} GB will spill to remote nodes (H2D may slow "
                f"~10-15%). Pass `numa_node=None` to let the kernel spread freely.",
                stacklevel=3,
            )

    def _master_source(self, p):
        """Full-shape tensor the fp32 master is seeded from."""
        return p.data

    def _seed_master(self, p, master):
        master.copy_(self._master_source(p))

    def _alloc_pinned_states(self, params, numa_node):
        specs, where = [], []
        for p in params:
            for key, dtype in self.offload_config.items():
                specs.append((self._state_shape(p, key), dtype))
                where.append((p, key))
        if not specs:
            return
        tensors = self._make_host_tensors(specs, numa_node)
        for (p, key), t in zip(where, tensors):
            self.state[p][key] = t
        for p in params:
            st = self.state[p]
            if self._has_master:
                self._seed_master(p, st["master_params"])
                if p in self._quant_params:
                    st["master_filled"] = False
        if self.verbose > 0:
            total = sum(t.numel() * t.element_size() for t in tensors)
            print(f"{self._log_prefix()}Pinned host memory allocated: {total / 1024**3:.2f} GB")

    def _log_prefix(self):
        return ""

    def _make_host_tensors(self, specs, numa_node):
        if self._cuda:
            self._arena = PinnedArena(specs, numa_node=numa_node, device=self.device)
            if self.verbose > 0:
                s = self._arena.stats()
                print(f"{self._log_prefix()}pinned arena: {s['segments']} segment(s), numa_node={s['numa_node']}, "
                      f"map {s['seconds_map']:.2f}s touch {s['seconds_touch']:.2f}s "
                      f"register {s['seconds_register']:.2f}s")
            return list(self._arena.tensors())
        return [torch.zeros(tuple(shape), dtype=dtype) for shape, dtype in specs]

    def _alloc_inplace_states(self, params):
        total = 0
        entries = []
        for p in self._all_params:
            if p not in params:
                continue
            st = self.state[p]
            for key, dtype in self.offload_config.items():
                t = torch.zeros_like(p, dtype=dtype)
                if key == "master_params":
                    t.copy_(p.data)
                st[key] = t
                total += t.numel() * t.element_size()
            extra = st.get("master_params", st.get("rounding_error"))
            entries.append({"param": p.data, "grad": st["grad"], "exp_avg": st["exp_avg"],
                            "exp_avg_sq": st["exp_avg_sq"], "extra": extra, "p": p})
        self._inplace_entries = entries
        if self.verbose > 0 and entries:
            print(f"{self._log_prefix()}In-place GPU states for {len(entries)} small params: "
                  f"{total / 1024**2:.2f} MB")

    # ------------------------------------------------------------ hook bodies
    def _resolve_staging_bytes(self, staging_bytes):
        # the state itself plus the padding of its tensors: with that much everything can
        # stay resident, and more buys nothing
        state = self._estimate_pinned_bytes(self._offload_params) + 768 * len(self._offload_params)
        if staging_bytes is None:
            staging_bytes = state
            if self._cuda:
                # a quarter of the device, but never more than a third of what is free
                # now (the model is already resident; activations still need room)
                free, total = torch.cuda.mem_get_info(self.device)
                staging_bytes = min(state, total // 4, max(free // 3, 1 << 30))
        return min(int(staging_bytes), state)

    def _hp(self, group):
        b1, b2 = group["betas"]
        return (group["lr"], group["weight_decay"], b1, b2, group["eps"])

    def _slot(self, p):
        i = self._pid[p]
        return self._normsq[i : i + 1]

    def _want_norm(self):
        return self.max_grad_norm is not None and self.ready_for_optimizer_step

    def _take_grad(self, p):
        g = p.grad
        p.grad = None
        if g.dtype != _BF16 or not g.is_contiguous():
            g = g.to(_BF16).contiguous()
        return g

    @torch.no_grad()
    def _grad_hook(self, p):
        if not self._nvtx:
            return self._grad_hook_body(p)
        torch.cuda.nvtx.range_push("oab.grad_hook")
        try:
            return self._grad_hook_body(p)
        finally:
            torch.cuda.nvtx.range_pop()

    def _grad_hook_body(self, p):
        if p.grad is None:
            return
        self._pace_prefetch(1)
        grad = self._take_grad(p)
        st = self.state[p]
        last = self.ready_for_optimizer_step
        sumsq = self._slot(p) if self._want_norm() else None
        if self.grad_residency == "device":
            acc = self._dev_grad.get(p)
            if acc is None:
                self._dev_grad[p] = grad
                if sumsq is not None:
                    grad_ops.grad_accumulate(None, grad, None, sumsq=sumsq, scratch=self._scratch_main)
            else:
                grad_ops.grad_accumulate(acc, acc, grad, sumsq=sumsq, scratch=self._scratch_main)
            if last and self._step_in_backward:
                self._step_offload(p, self._param2group[p])
            return
        # ---- host residency
        if last and self._step_in_backward:
            self._step_offload(p, self._param2group[p], dev_grad=grad)
            return
        self._engine.grad_to_host(self._pid[p], st["grad"], grad, first=not st["host_grad_valid"],
                                  sumsq=sumsq)
        st["host_grad_valid"] = True

    @torch.no_grad()
    def _inplace_grad_hook(self, p):
        if p.grad is None:
            return
        grad = self._take_grad(p)
        st = self.state[p]
        sumsq = self._slot(p) if self._want_norm() else None
        grad_ops.grad_accumulate(st["grad"], st["grad"], grad, sumsq=sumsq, scratch=self._scratch_main)
        if self.ready_for_optimizer_step and self._step_in_backward:
            st["step"] += 1
            self._pending_inplace.append(p)

    # ------------------------------------------------------------- step pieces
    def _param_view(self, p):
        """bf16 tensor the kernel writes the updated parameter into."""
        return p.data

    def _after_param_update(self, p):
        """Hook for subclasses (e.g. all-gather of an updated shard)."""

    def _grad_is_persistent(self, p):
        """True when the gradient handed to the step lives in a buffer the optimizer owns for
        good (nothing to keep alive, nothing to count against the gradient budget)."""
        return False

    def _step_extra(self, p):
        """Extra keyword arguments of ``TransferEngine.step`` (peer addresses)."""
        return {}

    def _step_offload(self, p, group, clip_coef=None, dev_grad=None, fork=True):
        """Enqueue the step of one offloaded parameter on the side streams.  ``fork=False``:
        the optimizer stream is already ordered after the main stream (the caller forked it
        and has put nothing on the main stream since)."""
        st = self.state[p]
        st["step"] += 1
        self._step_dirty = True
        if self._step_in_backward:
            self._hook_order_cur.append(p)
        if dev_grad is None:
            dev_grad = self._dev_grad.pop(p, None)
        host_grad = st["grad"] if st["host_grad_valid"] else None
        extra = self._step_extra(p)
        if dev_grad is None and host_grad is None and not extra.get("g_peers"):
            st["step"] -= 1
            return
        seed = self._rng.getrandbits(63) if self.mode == "stochastic_rounding" else 0
        states = {k: st[k] for k in self._non_grad_keys}
        quant = p in self._quant_params
        if quant:
            self._warn_lossy_master_once(st)
            self._step_quant(p, group, st, dev_grad, host_grad, clip_coef, fork=fork)
        else:
            self._engine.step(self._pid[p], self._param_view(p), dev_grad, host_grad, states,
                              self._hp(group), st["step"], self.decoupled_weight_decay,
                              clip=clip_coef, seed=seed, fork=fork,
                              retain=not self._grad_is_persistent(p), **extra)
        st["host_grad_valid"] = False
        self._after_param_update(p)

    # ------------------------------------------------------- quantized weights
    def _quant_replicas(self, p):
        """``(row0, payload0 addresses, payload1 addresses)``: which rows of the weight this
        optimizer updates and where their packed form goes (subclasses add the other
        ranks' replicas)."""
        a, b = p.KERNEL_PAYLOAD
        return 0, [getattr(p, a).data_ptr()], [getattr(p, b).data_ptr()]

    def _fused_quant_ok(self, p):
        return self._fused_quant_plan(p) is not None

    def _fused_quant_plan(self, p):
        """How quantized parameter ``p`` is stepped: a dict for the fused route (Adam on the
        master chunk by chunk through the staging buffer, re-quantization and the store of
        the packed rows in the same pass) or None for the unfused one (CPU tensors, shapes
        the kernels do not take, ``transfer='zero_copy'``)."""
        if p in self._fused_quant:
            return self._fused_quant[p]
        plan = None
        eng = self._engine
        C = getattr(eng, "C", None)
        scale_ids = None if C is None else {torch.float32: C.QDT_F32, torch.bfloat16: C.QDT_BF16,
                                            torch.float16: C.QDT_F16}
        if (self._cuda and eng._native is not None and p.KERNEL_FORMAT and p.dim() == 2
                and p.kernel_scale_dtype() in scale_ids
                and C.adam_quant_supported(p.KERNEL_FORMAT, p.shape[1], p.kernel_group())
                and all(getattr(p, k).is_contiguous() for k in p.KERNEL_PAYLOAD)):
            in_f = p.shape[1]
            rows = max(1, eng.chunk_elems // in_f)
            if rows >= 32:
                rows = rows // 32 * 32  # whole 32-row tiles for the transposed int4 payload
            row0, pay0, pay1 = self._quant_replicas(p)
            nvfp4 = bool(p.USES_TENSOR_AMAX)
            if nvfp4 and self._amax is None:
                self._amax = torch.zeros(2 * len(self._all_params), dtype=torch.float32, device=self.device)
            i = self._pid[p]
            local_amax = self._amax[2 * i: 2 * i + 1] if nvfp4 else None
            tensor_amax = self._amax[2 * i + 1: 2 * i + 2] if (nvfp4 and self._quant_amax_is_global(p)) else local_amax
            spec = C.QuantSpec(p.KERNEL_FORMAT, p.shape[0], in_f, row0, p.kernel_group(),
                               scale_ids[p.kernel_scale_dtype()], pay0, pay1, tensor_amax,
                               p.global_scale if nvfp4 else None)
            plan = {"chunk": rows * in_f, "spec": spec, "nvfp4": nvfp4, "local_amax": local_amax,
                    "tensor_amax": tensor_amax}
        self._fused_quant[p] = plan
        return plan

    def _quant_amax_is_global(self, p):
        """True when max|master| of ``p`` has to be combined across ranks first."""
        return False

    def _chunk_for(self, p):
        """Chunk length of ``p`` in the staging buffer (0: the engine's default)."""
        if p not in self._quant_params:
            return 0
        plan = self._fused_quant_plan(p)
        return plan["chunk"] if plan else 0

    def _combine_amax(self, p, plan):
        """Hook for subclasses: turn the local max|master| into the whole weight's."""

    def _step_quant(self, p, group, st, dev_grad, host_grad, clip_coef, fork=True):
        """Quantized parameter on the fused route: the fp32 master and the moments stream
        through the staging buffer like any dense tensor; each chunk is a number of whole
        rows, and the kernel that updates them also re-quantizes them and stores the packed
        rows (reference: src/offload_adam/offload_adam.py:421-444 keeps the whole master on
        the GPU and re-quantizes it with a second kernel)."""
        plan = self._fused_quant_plan(p)
        if plan is None:
            return self._step_quant_unfused(p, group, st, dev_grad, host_grad, clip_coef)
        eng = self._engine
        states = {k: st[k] for k in self._non_grad_keys}
        extra = {k: v for k, v in self._step_extra(p).items() if k != "p_peers"}
        n = states["exp_avg"].numel()
        tmp = None
        if plan["nvfp4"] and not eng.is_resident(self._pid[p]):
            if self._master_tmp is None or self._master_tmp.numel() < n:
                need = max(self._state_elems(q) for q in self._quant_params if q.USES_TENSOR_AMAX)
                self._master_tmp = torch.empty(need, dtype=torch.float32, device=self.device)
            tmp = self._master_tmp
        where = eng.step(self._pid[p], None, dev_grad, host_grad, states, self._hp(group), st["step"],
                         self.decoupled_weight_decay, clip=clip_coef, amax=plan["local_amax"],
                         quant=plan["spec"], chunk=plan["chunk"], master_copy=tmp, fork=fork,
                         retain=not self._grad_is_persistent(p), **extra)
        if plan["nvfp4"]:
            # second pass: the tensor scale needs max|master| of the whole updated weight
            self._combine_amax(p, plan)
            eng.C.nvfp4_quantize_push(plan["spec"], where, n, extra.get("status"), eng.opt_stream.cuda_stream)
            if eng.serialize:
                eng.synchronize()

    def _step_quant_unfused(self, p, group, st, dev_grad, host_grad, clip_coef):
        """Quantized parameter without the fused kernels: the fp32 master makes the round
        trip through a device temporary and a separate kernel (or, on CPU tensors, the
        PyTorch restatement) re-quantizes it."""
        eng = self._engine
        if not self._cuda:
            states = {k: st[k] for k in self._non_grad_keys}
            eng.step(self._pid[p], None, dev_grad, host_grad, states, self._hp(group), st["step"],
                     self.decoupled_weight_decay, clip=clip_coef)
            p.data.copy_(st["master_params"])
            return
        eng.fork_from_main()
        with torch.cuda.stream(eng.opt_stream):
            master = st["master_params"].to(self.device, non_blocking=True)
            states = {"exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"], "master_params": master}
            g = dev_grad if dev_grad is not None else host_grad
            g2 = host_grad if dev_grad is not None else None
            states["grad"] = g
            # formats with a per-tensor scale get max|master| as a by-product of the step
            amax = torch.zeros(1, dtype=torch.float32, device=self.device) \
                if getattr(p.data, "USES_TENSOR_AMAX", False) else None
            adam_step(self.mode, None, states, *self._hp(group), st["step"],
                      decoupled_weight_decay=self.decoupled_weight_decay, clip_coef=clip_coef,
                      grad2=g2, amax=amax, max_ctas=eng.max_ctas, stream=eng.opt_stream.cuda_stream,
                      use_cuda=True)
            if amax is not None:
                p.data._quantize_into(master, amax)
            else:
                p.data.copy_(master)
            st["master_params"].copy_(master, non_blocking=True)
        eng._retain(dev_grad)

    def _step_inplace_batch(self, params, clip_coef=None):
        """One multi-tensor launch for the small GPU-resident parameters."""
        if not params:
            return
        group0 = self._param2group[params[0]]
        same = all(self._param2group[p] is group0 for p in params) and \
            len({self.state[p]["step"] for p in params}) == 1
        seed = self._rng.getrandbits(63) if self.mode == "stochastic_rounding" else 0
        if same and len(params) == len(self._inplace_entries) and len(self.param_groups) == 1:
            if self._multi is None:
                self._multi = grad_ops.MultiTensorAdam(self._inplace_entries, self.mode)
            lr, wd, b1, b2, eps = self._hp(group0)
            self._multi.step(lr, wd, b1, b2, eps, self.state[params[0]]["step"],
                             self.decoupled_weight_decay, clip_coef=clip_coef, seed=seed,
                             zero_grad=True)
            return
        entry = {e["p"]: e for e in self._inplace_entries}
        for p in params:
            st = self.state[p]
            tensors = {k: st[k] for k in self.offload_state_keys}
            tensors["grad"] = entry[p]["grad"]  # subclasses may step from a reduced copy
            adam_step(self.mode, p.data, tensors, *self._hp(self._param2group[p]), st["step"],
                      decoupled_weight_decay=self.decoupled_weight_decay, clip_coef=clip_coef,
                      seed=self._rng.getrandbits(63))
            tensors["grad"].zero_()

    def _on_forward(self):
        self._finish_step()
        self._pace_prefetch(1)

    def _start_prefetch(self):
        """Begin a new round of early H2D for the step that has just started.  Order:
        parameter order on the clipping path, the hook order of the previous step
        otherwise."""
        self._pf_order, self._pf_idx, self._pf_off = None, 0, 0
        eng = self._engine
        if not (self._cuda and eng.can_prefetch and self.grad_residency == "device"):
            return
        order = self._step_order_guess()
        if self.prefetch_pacing == "thread" and self.prefetch_inflight > 0:
            items = []
            for p in order or ():
                if p in self._quant_params and self._fused_quant_plan(p) is None:
                    break  # takes its own route through a device temporary
                st = self.state[p]
                items.append((self._pid[p], {k: st[k] for k in self._non_grad_keys}, self._chunk_for(p)))
            eng.start_prefetch(items, self.prefetch_inflight)
            return
        self._pf_order = order or None

    def _pace_prefetch(self, max_chunks):
        """Issue a few more chunks of early H2D.  Called from the forward pre-hook and
        from every gradient hook: the bulk copies are spread over the step instead of
        being queued at once, so copies of the caller (input batches) never wait behind
        more than a few chunks in the copy engine."""
        order = self._pf_order
        if order is None:
            return
        eng = self._engine
        inflight = self.prefetch_inflight
        budget = max_chunks if inflight > 0 else 1 << 30  # unbounded: everything that fits, at once
        while budget > 0:
            if self._pf_idx >= len(order):
                self._pf_order = None
                return
            p = order[self._pf_idx]
            if p in self._quant_params and self._fused_quant_plan(p) is None:
                self._pf_order = None  # takes its own route through a device temporary
                return
            st = self.state[p]
            states = {k: st[k] for k in self._non_grad_keys}
            off, full = eng.prefetch(self._pid[p], states, None, self._pf_off, budget, max_inflight=inflight,
                                     chunk=self._chunk_for(p))
            if full:
                self._pf_order = None  # no staging space left for this step
                return
            issued = -(-(off - self._pf_off) // (self._chunk_for(p) or eng.chunk_elems))
            if off >= states["exp_avg"].numel():
                self._pf_idx += 1
                self._pf_off = 0
            else:
                self._pf_off = off
            if issued == 0:
                return  # earlier copies are still in flight
            budget -= issued

    def _finish_step(self):
        """Run what the hooks deferred and make the main stream wait for the side
        streams.  Idempotent; called by ``step()`` and before every forward."""
        if self._pending_inplace:
            pend, self._pending_inplace = self._pending_inplace, []
            self._step_inplace_batch(pend)
        if self._step_dirty:
            # only a finished step forces the join: gradient write-backs of earlier
            # micro-batches keep overlapping the next forward
            self._step_dirty = False
            self._engine.join_main(wait_writeback=False)
            self._hook_order_prev, self._hook_order_cur = (self._hook_order_cur or self._hook_order_prev), []
            self._start_prefetch()

    # -------------------------------------------------------------- public API
    @torch.no_grad()
    def step(self, closure=None):
        if not self._nvtx:
            return self._step_body(closure)
        torch.cuda.nvtx.range_push("oab.step")
        try:
            return self._step_body(closure)
        finally:
            torch.cuda.nvtx.range_pop()

    def _step_body(self, closure=None):
        if closure is not None:
            raise NotImplementedError(
                f"{type(self).__name__} does not support closure-based step: gradients are "
                "consumed by backward hooks, so re-running backward inside a closure would "
                "corrupt optimizer state."
            )
        if self._step_in_backward:
            self._finish_step()
            return
        self._engine.stop_prefetch()
        if self.verbose > 1 and self._engine.can_prefetch:
            nat = self._engine._native
            print(f"{self._log_prefix()}step: {nat.prefetched_chunks()} chunk(s), "
                  f"{nat.prefetched_bytes() / 2**30:.2f} of {nat.ring_bytes() / 2**30:.2f} GiB of staging "
                  f"hold prefetched state", flush=True)
        trace = self.verbose > 2
        eng = self._engine
        if trace:
            eng.begin_trace()
            eng.mark("step_begin")
            eng.mark("earlier_loads_done", "h2d")
            eng.mark("earlier_writebacks_done", "d2h")
        clip = self._global_clip_coef()
        if trace:
            eng.mark("clip_coef_done")
        inplace = []
        # one fork serves the whole loop: nothing lands on the main stream inside it
        self._engine.fork_from_main()
        host_t = [time.perf_counter()] if trace else None
        for group in self.param_groups:
            for p in group["params"]:
                if p in self._inplace_params:
                    self.state[p]["step"] += 1
                    inplace.append(p)
                else:
                    self._step_offload(p, group, clip_coef=clip, fork=False)
        if trace:
            host_t.append(time.perf_counter())
        self._step_inplace_batch(inplace, clip_coef=clip)
        if trace:
            eng.mark("kernels_done", "opt")
            eng.mark("loads_done", "h2d")
            eng.mark("writebacks_done", "d2h")
        self._finish_step()
        if trace:
            eng.mark("step_end")
            host_t.append(time.perf_counter())
            self.host_trace = {"enqueue_all_tensors_ms": round((host_t[1] - host_t[0]) * 1e3, 2),
                               "small_tensors_and_finish_ms": round((host_t[2] - host_t[1]) * 1e3, 2)}
        if self.max_grad_norm is not None:
            torch.sqrt(self._normsq, out=self._norms)
            self._normsq.zero_()

    def _global_clip_coef(self):
        """Device scalar min(1, max_norm / (||g|| + 1e-6)); no host sync."""
        if self.max_grad_norm is None:
            return None
        # squared norms were written by kernels on the optimizer stream (host residency)
        # or on the main stream (device residency); order the reduction after both.
        # Copies still in flight (early loads, trailing write-backs) are not waited for.
        self._engine.join_main(wait_writeback=False)
        grad_ops.clip_finalize(self._normsq, None, None, self.max_grad_norm, coef_norm=self._clip)
        return self._clip[0:1]

    def zero_grad(self, set_to_none=False):
        """No-op: gradients are consumed and cleared by the hooks."""
        return

    def state_dict(self):
        """Same layout as the reference; waits for write-backs still in flight first."""
        self.synchronize()
        return super().state_dict()

    def trace_report(self, current=True):
        """Timeline of the last one-shot ``step()`` taken with ``verbose`` > 2 (see
        ``TransferEngine.mark``): milliseconds from the start of the step to named points
        on the main, optimizer, H2D and D2H streams.  ``None`` until the step's work has
        completed; never blocks."""
        return self._engine.trace_report(current)

    def synchronize(self):
        """Block the host until every enqueued transfer and step has finished."""
        self._finish_step()
        self._engine.synchronize()

    def memory_report(self):
        """Bytes this optimizer holds, by place: ``pinned_host`` (state of the offloaded
        parameters, and their gradient buffers under host residency), ``device_state``
        (state of the small parameters kept on the GPU), ``device_staging`` (the staging
        buffer of the staged transfer) and ``device_grad_accumulators`` (bf16 gradient
        accumulators alive right now under device residency)."""
        def nbytes(t):
            return t.numel() * t.element_size()

        pinned = device_state = 0
        for p in self._all_params:
            for v in self.state[p].values():
                if isinstance(v, torch.Tensor) and v.dim() > 0:
                    if p in self._inplace_params:
                        device_state += nbytes(v)
                    else:
                        pinned += nbytes(v)
        return {"pinned_host": pinned, "device_state": device_state,
                "device_staging": int(self._engine.staging_bytes),
                "device_grad_accumulators": sum(nbytes(g) for g in self._dev_grad.values())}

    def close(self):
        """Detach from the model: finish everything in flight and remove the hooks, so
        that gradients reach ``p.grad`` again (for instance before building another
        optimizer for the same model).  The state stays readable through
        ``state_dict()``; stepping a closed optimizer is an error of the caller."""
        self.synchronize()
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []

    def __del__(self):
        # transfers in flight still touch the pinned state and the staging buffer:
        # finish them before either is released
        eng = getattr(self, "_engine", None)
        if eng is not None and getattr(self, "_owner_pid", None) == os.getpid():  # not in a forked child
            try:
                eng.synchronize()
            except Exception:
                pass

    def wait_writeback(self):
        """Block the host until the optimizer state of the last step is back in host
        memory (it normally drains behind the next forward pass).  Early loads of the
        next step keep running, unlike with ``synchronize()``."""
        self._engine.wait_writeback()

    def _copy_master(self, p, tensor):
        self._engine.invalidate_prefetched()  # a copy loaded ahead of time would be stale
        self.state[p]["master_params"].copy_(tensor)

    def _tracks(self, p):
        return p in self.state

    def load_state_dict(self, state_dict):
        raise NotImplementedError(
            f"{type(self).__name__}.load_state_dict is not supported: the default "
            "Optimizer.load_state_dict would move pinned-host state to GPU and cast the fp32 "
            "master to bf16, defeating the offload contract. Use load_offload_state_dict() to "
            "resume into the existing pinned buffers."
        )

    @torch.no_grad()
    def load_offload_state_dict(self, state_dict):
        """Resume from ``state_dict()`` output by copying into the existing buffers
        (pinned host tensors stay where they are, dtypes are preserved)."""
        self.synchronize()
        self._engine.invalidate_prefetched()  # state loaded ahead of time would be stale
        saved_ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        live = [p for g in self.param_groups for p in g["params"]]
        if len(saved_ids) != len(live):
            raise ValueError("load_offload_state_dict: parameter count differs from the checkpoint")
        for g_live, g_saved in zip(self.param_groups, state_dict["param_groups"]):
            for k, v in g_saved.items():
                if k != "params":
                    g_live[k] = v
        for idx, p in zip(saved_ids, live):
            src = state_dict["state"].get(idx)
            if src is None:
                continue
            dst = self.state[p]
            for k, v in src.items():
                if isinstance(v, torch.Tensor) and isinstance(dst.get(k), torch.Tensor):
                    if k == "grad":
                        continue  # transient accumulator, never part of a resume
                    if v.shape != dst[k].shape or v.dtype != dst[k].dtype:
                        raise ValueError(f"load_offload_state_dict: state '{k}' of param {idx} "
                                         f"has shape/dtype {tuple(v.shape)}/{v.dtype}, expected "
                                         f"{tuple(dst[k].shape)}/{dst[k].dtype}")
                    dst[k].copy_(v)
                elif k == "host_grad_valid":
                    continue  # goes with the gradient buffer, which is not restored
                else:
                    dst[k] = v
            if "host_grad_valid" in dst:
                dst["host_grad_valid"] = False
        self._dev_grad.clear()
