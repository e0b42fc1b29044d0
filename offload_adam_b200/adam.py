"""``Adam``: the non-offloaded bf16-aware Adam/AdamW baseline.

Same four parameter-precision modes and the same state layout as the offloaded
optimizers, with every tensor resident on the parameter's device
(reference: src/offload_adam/adam.py:16-302).  State per parameter: ``step``
(int), ``exp_avg`` / ``exp_avg_sq`` (bf16, bias-corrected moments), and by mode
``master_params`` (fp32) or ``rounding_error`` (int16); quantized parameters
additionally carry ``master_filled`` (bool).
"""

from __future__ import annotations

import random

import torch
from torch.optim.optimizer import Optimizer

from ._master import MasterLoadingMixin, is_quant
from .ops.adam_step import STEP_FNS

STATE_DTYPES = {
    "stochastic_rounding": {"exp_avg": torch.bfloat16, "exp_avg_sq": torch.bfloat16},
    "fp32_master": {
        "exp_avg": torch.bfloat16,
        "exp_avg_sq": torch.bfloat16,
        "master_params": torch.float32,
    },
    "fp31_master": {
        "exp_avg": torch.bfloat16,
        "exp_avg_sq": torch.bfloat16,
        "rounding_error": torch.int16,
    },
    "fp32_master_custom_rounding": {
        "exp_avg": torch.bfloat16,
        "exp_avg_sq": torch.bfloat16,
        "rounding_error": torch.int16,
    },
}


class Adam(MasterLoadingMixin, Optimizer):
    """Adam / AdamW for bf16 parameters with state on the parameter's device.

    Args:
        params: iterable of parameters or param groups.
        lr, betas, eps, weight_decay: the usual Adam hyper-parameters.
        mode: ``'stochastic_rounding'`` (default), ``'fp32_master'``,
            ``'fp31_master'`` or ``'fp32_master_custom_rounding'``.
        decoupled_weight_decay: AdamW-style decay when True.
        seed: seeds the stochastic-rounding stream (default: Python's ``random``).
    """

    configs = {k: {"step": STEP_FNS[k], "states": v} for k, v in STATE_DTYPES.items()}

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 mode="stochastic_rounding", decoupled_weight_decay=False, seed=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        assert mode in self.configs, f"Invalid mode: {mode}"
        self.mode = mode
        self.config = self.configs[mode]
        self.step_fn = self.config["step"]
        self.decoupled_weight_decay = decoupled_weight_decay
        self._has_master = "master_params" in self.config["states"]
        self._rng = random.Random(seed)
        n_quant = sum(1 for g in self.param_groups for p in g["params"] if is_quant(p))
        if n_quant and mode != "fp32_master":
            raise ValueError(
                f"Adam found {n_quant} quantized param(s) but mode={mode!r}; "
                f"QAT requires mode='fp32_master'."
            )
        # nothing to warn about when there is no quantized parameter
        self._quant_master_warned = n_quant == 0

    # ------------------------------------------------------------------ state
    def _init_state_if_empty(self, p, state):
        if state:
            return
        state["step"] = 0
        for name, dtype in self.config["states"].items():
            state[name] = torch.zeros_like(p, dtype=dtype)
        if self._has_master:
            # dense param: exact widening; quantized param: dequantized (lossy) seed
            state["master_params"].copy_(p.data)
            if is_quant(p):
                state["master_filled"] = False

    def _copy_master(self, p, tensor):
        self.state[p]["master_params"].copy_(tensor)

    # ------------------------------------------------------------------- step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                grad = p.grad
                if grad is None:
                    continue
                if grad.is_sparse:
                    raise RuntimeError("Sparse gradient is not supported")
                state = self.state[p]
                self._init_state_if_empty(p, state)
                state["step"] += 1
                quant = is_quant(p)
                if quant:
                    self._warn_lossy_master_once(state)
                tensors = {k: state[k] for k in self.config["states"]}
                tensors["grad"] = grad if grad.dtype == torch.bfloat16 else grad.to(torch.bfloat16)
                kw = {}
                if self.mode == "stochastic_rounding":
                    kw["seed"] = self._rng.getrandbits(63)
                # a quantized weight has no bf16 image to write: only the master moves,
                # then copy_ re-quantizes the packed payload from it
                self.step_fn(
                    None if quant else p.data, tensors, group["lr"], group["weight_decay"], beta1,
                    beta2, group["eps"], state["step"],
                    decoupled_weight_decay=self.decoupled_weight_decay, **kw,
                )
                if quant:
                    p.data.copy_(state["master_params"])
                    p.grad = None
        return loss

    # ------------------------------------------------------------- checkpoint
    @torch.no_grad()
    def load_state_dict(self, state_dict):
        """``Optimizer.load_state_dict`` casts floating state to the parameter's
        dtype, which would demote the fp32 master to bf16; put the original fp32
        tensors back afterwards."""
        keep = {}
        for idx, st in state_dict.get("state", {}).items():
            t = st.get("master_params") if isinstance(st, dict) else None
            if isinstance(t, torch.Tensor) and t.dtype == torch.float32:
                keep[idx] = t.detach()
        super().load_state_dict(state_dict)
        if not keep:
            return
        # state_dict indices follow the order of params across groups
        saved_ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        live = [p for g in self.param_groups for p in g["params"]]
        for idx, p in zip(saved_ids, live):
            if idx in keep and "master_params" in self.state.get(p, {}):
                self.state[p]["master_params"] = keep[idx].to(device=p.device).clone()
