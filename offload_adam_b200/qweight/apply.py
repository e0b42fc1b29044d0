"""Model surgery for QAT: swap ``nn.Linear`` weights for quantized tensor subclasses
and keep checkpoints in plain tensors.

``quantize_linears`` replaces the weight ``Parameter`` of every eligible linear
layer by a ``weight_cls`` instance and installs two ``state_dict`` hooks on the
layer: on save the subclass is expanded into the format's canonical plain tensors
(safetensors / ``weights_only=True`` friendly); on load those tensors are folded
back into a subclass instance, while a dense ``weight`` in the checkpoint is left
alone so that ``copy_`` re-quantizes it
(reference: src/offload_adam/qweight/apply.py:17-187).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import List, NamedTuple, Optional, Tuple, Type, Union

import torch
import torch.nn as nn

from .base import QWeightBase


class QuantizeReport(NamedTuple):
    """Module names (as in ``model.named_modules()``) by outcome of a
    ``quantize_linears`` pass: ``quantized``; ``incompatible`` as
    ``(name, reason)`` pairs rejected by ``can_quantize``; ``excluded`` by
    ``skip_patterns``."""

    quantized: List[str]
    incompatible: List[Tuple[str, str]]
    excluded: List[str]


def _install_state_dict_hooks(module: nn.Module, weight_cls: Type[QWeightBase]) -> None:
    suffixes = weight_cls.canonical_key_suffixes()

    def on_save(mod, destination, prefix, local_metadata):
        w = destination.get(prefix + "weight")
        if isinstance(w, weight_cls):
            del destination[prefix + "weight"]
            for suffix, tensor in w.to_plain_state_dict().items():
                destination[prefix + suffix] = tensor

    def before_load(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        found = {s: state_dict.pop(prefix + s) for s in suffixes if prefix + s in state_dict}
        # NF4 names its packed bytes "weight" too: a non-uint8 "weight" is a dense
        # checkpoint tensor and goes back for copy_ to re-quantize
        dense = found.get("weight")
        if dense is not None and dense.dtype is not torch.uint8:
            state_dict[prefix + "weight"] = found.pop("weight")
        if not found:
            return
        if len(found) < len(suffixes):
            missing_keys.extend(prefix + s for s in suffixes if s not in found)
            return
        current = module.weight.data
        state_dict[prefix + "weight"] = weight_cls.from_plain_state_dict(
            found, reference=current if isinstance(current, weight_cls) else None)

    module._register_state_dict_hook(on_save)
    module._register_load_state_dict_pre_hook(before_load)


@torch.no_grad()
def quantize_linears(model: nn.Module, weight_cls: Type[QWeightBase], skip_patterns: Tuple[str, ...] = (),
                     device: Optional[str] = None, strict: bool = False, update_hf_config: bool = False,
                     **weight_kwargs) -> QuantizeReport:
    """Quantize eligible ``nn.Linear`` weights of ``model`` in place.

    Args:
        weight_cls: format class providing ``from_float`` / ``can_quantize``.
        skip_patterns: substrings; a layer whose qualified name contains one is
            reported under ``excluded`` and left dense (e.g. ``("lm_head",)``).
        device: move each weight there before quantizing.
        strict: raise ``ValueError`` if ``can_quantize`` rejects any layer.
        update_hf_config: set ``model.config.quantization_config`` when the model
            has a ``config`` attribute.
        **weight_kwargs: forwarded to ``from_float`` and ``can_quantize``
            (``group_size=``, ``blocksize=``, ...).
    """
    report = QuantizeReport([], [], [])
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear):
            continue
        if any(pat in name for pat in skip_patterns):
            report.excluded.append(name)
            continue
        old = module.weight
        if not weight_cls.can_quantize(old, **weight_kwargs):
            report.incompatible.append((name, f"shape={tuple(old.shape)} dtype={old.dtype}"))
            continue
        dense = old.data if device is None else old.data.to(device)
        module.weight = nn.Parameter(weight_cls.from_float(dense, **weight_kwargs), requires_grad=old.requires_grad)
        _install_state_dict_hooks(module, weight_cls)
        report.quantized.append(name)
    if strict and report.incompatible:
        detail = "; ".join(f"{n} ({r})" for n, r in report.incompatible)
        raise ValueError(f"quantize_linears(strict=True) rejected {len(report.incompatible)} layer(s): {detail}")
    if update_hf_config and hasattr(model, "config"):
        model.config.quantization_config = weight_cls.build_hf_quantization_config(
            skip_patterns=skip_patterns, **weight_kwargs)
    return report


def save_quantized_pretrained(model: nn.Module, save_directory: Union[str, Path], weight_cls: Type[QWeightBase],
                              skip_patterns: Tuple[str, ...] = (), **weight_kwargs) -> None:
    """``model.save_pretrained(save_directory)`` followed by writing the format's
    ``quantization_config`` into the saved ``config.json``."""
    out = Path(save_directory)
    model.save_pretrained(out)
    cfg_file = out / "config.json"
    cfg = json.loads(cfg_file.read_text())
    cfg["quantization_config"] = weight_cls.build_hf_quantization_config(skip_patterns=skip_patterns, **weight_kwargs)
    cfg_file.write_text(json.dumps(cfg, indent=2))
