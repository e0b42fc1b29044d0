"""Gradient ops: bf16 accumulate fused with the squared-norm reduction, clip
coefficient, and the one-launch update of all small GPU-resident tensors.

They replace ``device_grad.add_(p.grad)``, ``torch.norm(grad)``, the
stack + vector_norm + clamp sequence and the per-tensor in-place step of the
reference (reference: src/offload_adam/offload_adam.py:398, :505, :555-561,
:456-467).
"""

from __future__ import annotations

import torch

from .. import _ext
from . import oracle
from .oracle import MODE_IDS, beta_hat


def sumsq_scratch(device) -> torch.Tensor:
    """Zeroed scratch area for the two-stage deterministic norm reduction."""
    device = torch.device(device)
    if device.type != "cuda":
        return torch.zeros(1, dtype=torch.float32, device=device)
    C = _ext.load(required=True)
    return torch.zeros(C.sumsq_scratch_bytes() // 4, dtype=torch.float32, device=device)


def grad_accumulate(out, a, b=None, sumsq=None, sumsq_accumulate=False, scratch=None,
                    max_ctas=0, stream=0, use_cuda=None):
    """out = bf16(a + b); ``sumsq`` (fp32 scalar tensor) receives sum(out^2).

    ``out`` may be None (norm only), ``b`` may be None (copy / norm of ``a``).
    Operands may be pinned host tensors mapped into the device.
    """
    if use_cuda is None:
        use_cuda = any(t is not None and t.is_cuda for t in (out, a, b, sumsq))
    if use_cuda:
        C = _ext.load(required=True)
        C.grad_accumulate(out, a, b, sumsq, bool(sumsq_accumulate), scratch, int(max_ctas), int(stream))
        return
    s = oracle.grad_accumulate(out, a, b, want_sumsq=sumsq is not None)
    if sumsq is not None:
        if sumsq_accumulate:
            sumsq.add_(s.reshape(sumsq.shape))
        else:
            sumsq.copy_(s.reshape(sumsq.shape))


def clip_finalize(slots, index, extra_sq, max_norm, coef_norm=None, total_sq=None, stream=0):
    """total = extra_sq + sum(slots[index]); coef_norm = [min(1, max/(sqrt(total)+1e-6)), sqrt(total)]."""
    ref = slots if slots is not None else extra_sq
    if ref.is_cuda:
        C = _ext.load(required=True)
        C.clip_finalize(slots, index, extra_sq, float(max_norm), coef_norm, total_sq, int(stream))
        return
    total = torch.zeros((), dtype=torch.float32)
    if slots is not None:
        sel = slots if index is None else slots[index.long()]
        total = total + sel.float().sum()
    if extra_sq is not None:
        total = total + extra_sq.reshape(()).float()
    if total_sq is not None:
        total_sq.copy_(total.reshape(total_sq.shape))
    if coef_norm is not None:
        coef, norm = oracle.clip_coef_from_sq(total, max_norm)
        coef_norm[0] = coef
        coef_norm[1] = norm


class MultiTensorAdam:
    """One launch that steps every small, GPU-resident parameter.

    ``entries`` is a list of dicts with keys ``param, grad, exp_avg, exp_avg_sq``
    and optionally ``extra`` (fp32 master / int16 error).  The pointer table and
    the block map are built once; tensors must not be reallocated afterwards.
    """

    def __init__(self, entries, mode):
        self.mode_id = MODE_IDS[mode] if isinstance(mode, str) else int(mode)
        self.entries = entries
        self.device = entries[0]["param"].device if entries else torch.device("cpu")
        self._table = None
        self._block_map = None
        if entries and self.device.type == "cuda":
            C = _ext.load(required=True)
            chunk = C.multi_tensor_chunk()
            rows, bmap = [], []
            off = 0
            for i, e in enumerate(entries):
                n = e["param"].numel()
                ex = e.get("extra")
                rows.append([
                    e["param"].data_ptr(), e["grad"].data_ptr(), e["exp_avg"].data_ptr(),
                    e["exp_avg_sq"].data_ptr(), ex.data_ptr() if ex is not None else 0, n, off,
                ])
                for c in range((n + chunk - 1) // chunk):
                    bmap.append([i, c])
                off += (n + 7) // 8 * 8
            self._table = torch.tensor(rows, dtype=torch.int64, device=self.device)
            self._block_map = torch.tensor(bmap, dtype=torch.int32, device=self.device)

    def step(self, lr, weight_decay, beta1, beta2, eps, step, decoupled, clip_coef=None, seed=0,
             zero_grad=True, stream=0):
        if not self.entries:
            return
        b1h, b2h = beta_hat(beta1, step), beta_hat(beta2, step)
        if self._table is not None:
            C = _ext.load(required=True)
            C.multi_tensor_adam(self._table, self._block_map, self.mode_id, bool(decoupled),
                                float(lr), float(weight_decay), b1h, b2h, float(eps), clip_coef,
                                int(seed) & ((1 << 63) - 1), bool(zero_grad), int(stream))
            return
        off = 0
        for e in self.entries:
            oracle.adam_step(self.mode_id, e["param"], e["grad"], e["exp_avg"], e["exp_avg_sq"],
                             e.get("extra"), lr, weight_decay, b1h, b2h, eps, decoupled,
                             clip=clip_coef, seed=seed, elem_offset=off)
            if zero_grad:
                e["grad"].zero_()
            off += (e["param"].numel() + 7) // 8 * 8
