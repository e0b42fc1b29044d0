"""fp32 master maintenance shared by ``Adam`` and ``OffloadAdam``.

Both optimizers can overwrite their fp32 master copies either from an
in-memory mapping or by streaming a safetensors checkpoint
(reference: src/offload_adam/offload_adam.py:577-670, adam.py:182-278).
"""

from __future__ import annotations

import warnings

import torch

from ._pretrained import stream_master_from_pretrained
from .qweight.base import QWeightBase

_LOSSY_MASTER_MSG = (
    "{name}: quantized params running with a lossy dequant-seeded fp32 master. "
    "For higher precision, call `optim.load_master_from_pretrained("
    "pretrained_name_or_path, model)` with the same bf16/fp16 checkpoint "
    "`from_pretrained` used before `quantize_linears` ran."
)


def is_quant(p) -> bool:
    return isinstance(p.data, QWeightBase)


class MasterLoadingMixin:
    """Needs: ``self.state``, ``self.mode``, ``self._has_master`` and
    ``self._copy_master(p, tensor)``; optionally ``self._init_state_if_empty``."""

    _quant_master_warned = False

    def _warn_lossy_master_once(self, state):
        if self._quant_master_warned or state.get("master_filled") is not False:
            return
        warnings.warn(_LOSSY_MASTER_MSG.format(name=type(self).__name__), stacklevel=4)
        self._quant_master_warned = True

    def _require_master(self, what):
        if not self._has_master:
            raise RuntimeError(
                f"{what} requires a mode that maintains master_params "
                f"(mode='fp32_master'); current mode is {self.mode!r}."
            )

    @torch.no_grad()
    def load_master_state_dict(self, state_dict, model, strict=False):
        """Overwrite fp32 masters from ``{param_name: tensor}`` (any float dtype).

        Returns ``(unexpected_keys,)``; with ``strict=True`` unknown names raise
        ``ValueError``.  Params touched get ``master_filled=True`` when they
        carry that flag (quantized params).
        """
        self._require_master("load_master_state_dict")
        by_name = {n: p for n, p in model.named_parameters() if p.requires_grad}
        init = getattr(self, "_init_state_if_empty", None)
        unexpected = []
        for name, tensor in state_dict.items():
            p = by_name.get(name)
            if p is None or not self._tracks(p):
                unexpected.append(name)
                continue
            st = self.state[p]
            if init is not None:
                init(p, st)
            self._copy_master(p, tensor)
            if "master_filled" in st:
                st["master_filled"] = True
        if strict and unexpected:
            raise ValueError(
                f"load_master_state_dict(strict=True): no param matches "
                f"{len(unexpected)} key(s): {unexpected}"
            )
        return (unexpected,)

    @torch.no_grad()
    def load_master_from_pretrained(self, pretrained_name_or_path, model, *, strict=False):
        """Refill the fp32 master of every quantized param from a checkpoint
        (single safetensors file, sharded directory or hub id), one tensor at a
        time.  Returns the sorted names of quantized params with no match."""
        self._require_master("load_master_from_pretrained")
        return stream_master_from_pretrained(self, pretrained_name_or_path, model, strict=strict)

    def _tracks(self, p) -> bool:
        return True
