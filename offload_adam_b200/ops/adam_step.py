"""Fused Adam/AdamW step ops.

Public functions mirror the reference kernel package
(reference: src/offload_adam/kernels/__init__.py:5-15):
``adam_step_<mode>(params, states, lr, weight_decay, beta1, beta2, eps, step,
decoupled_weight_decay=False)`` with ``states`` a dict holding ``grad``,
``exp_avg``, ``exp_avg_sq`` and, by mode, ``master_params`` or
``rounding_error``.  CUDA tensors (and pinned host tensors mapped into the
device, for the zero-copy path) run the sm_100a kernel; CPU tensors run the fp32
PyTorch restatement in :mod:`offload_adam_b200.ops.oracle`.

Extra keyword arguments expose what the fused kernel can do beyond the
reference: ``clip_coef`` (device scalar applied in fp32), ``grad2`` (second
gradient term, added with bf16 rounding), ``elem_offset`` (keeps the stochastic
rounding stream independent of chunking), ``amax`` (running max of |master|),
``max_ctas`` and ``stream``.
"""

from __future__ import annotations

import random

import torch

from .. import _ext
from . import oracle
from .oracle import MODE_IDS, beta_hat

_EXTRA_KEY = {0: None, 1: "master_params", 2: "rounding_error", 3: "rounding_error"}


def _on_gpu(*tensors):
    return any(t is not None and t.is_cuda for t in tensors)


def adam_step(
    mode,
    params,
    states,
    lr,
    weight_decay,
    beta1,
    beta2,
    eps,
    step,
    decoupled_weight_decay=False,
    seed=None,
    clip_coef=None,
    grad2=None,
    elem_offset=0,
    amax=None,
    max_ctas=0,
    stream=0,
    use_cuda=None,
    g_peers=None,
    g_scale=1.0,
    p_peers=None,
    status=None,
):
    mode_id = MODE_IDS[mode] if isinstance(mode, str) else int(mode)
    b1h = beta_hat(beta1, step)
    b2h = beta_hat(beta2, step)
    extra_key = _EXTRA_KEY[mode_id]
    extra = states[extra_key] if extra_key else None
    if mode_id != 1:
        assert params is not None and params.dtype == torch.bfloat16, "params must be bfloat16"
    if mode_id == 0 and seed is None:
        seed = random.getrandbits(63)
    seed = int(seed or 0) & ((1 << 63) - 1)
    g, m, v = states.get("grad"), states["exp_avg"], states["exp_avg_sq"]
    if use_cuda is None:
        use_cuda = _on_gpu(params, g, m, v)
    if use_cuda:
        C = _ext.load(required=True)
        C.adam_step(
            mode_id, params, g, grad2, m, v, extra, float(lr), float(weight_decay), b1h, b2h,
            float(eps), bool(decoupled_weight_decay), clip_coef, seed, int(elem_offset), amax,
            int(max_ctas), int(stream), list(g_peers or ()), float(g_scale), list(p_peers or ()),
            status,
        )
    else:
        assert not g_peers and not p_peers, "peer-memory arguments need CUDA"
        oracle.adam_step(
            mode_id, params, g, m, v, extra, lr, weight_decay, b1h, b2h, eps,
            decoupled_weight_decay, clip=clip_coef, g2=grad2, seed=seed, elem_offset=elem_offset,
            amax=amax,
        )


def adam_step_stochastic_rounding(params, states, lr, weight_decay, beta1, beta2, eps, step,
                                  seed=None, decoupled_weight_decay=False, **kw):
    adam_step("stochastic_rounding", params, states, lr, weight_decay, beta1, beta2, eps, step,
              decoupled_weight_decay=decoupled_weight_decay, seed=seed, **kw)


def adam_step_fp32_master(params, states, lr, weight_decay, beta1, beta2, eps, step,
                          decoupled_weight_decay=False, **kw):
    adam_step("fp32_master", params, states, lr, weight_decay, beta1, beta2, eps, step,
              decoupled_weight_decay=decoupled_weight_decay, **kw)


def adam_step_fp31_master(params, states, lr, weight_decay, beta1, beta2, eps, step,
                          decoupled_weight_decay=False, **kw):
    adam_step("fp31_master", params, states, lr, weight_decay, beta1, beta2, eps, step,
              decoupled_weight_decay=decoupled_weight_decay, **kw)


def adam_step_fp32_master_custom_rounding(params, states, lr, weight_decay, beta1, beta2, eps,
                                          step, decoupled_weight_decay=False, **kw):
    adam_step("fp32_master_custom_rounding", params, states, lr, weight_decay, beta1, beta2, eps,
              step, decoupled_weight_decay=decoupled_weight_decay, **kw)


STEP_FNS = {
    "stochastic_rounding": adam_step_stochastic_rounding,
    "fp32_master": adam_step_fp32_master,
    "fp31_master": adam_step_fp31_master,
    "fp32_master_custom_rounding": adam_step_fp32_master_custom_rounding,
}
