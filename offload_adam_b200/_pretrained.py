"""Stream fp32 masters of quantized params out of a safetensors checkpoint.

Accepts what ``from_pretrained`` accepts: one ``.safetensors`` file, a directory
(sharded with ``model.safetensors.index.json``, a single ``model.safetensors``,
or any ``*.safetensors``), or a hub repo id resolved with ``huggingface_hub``
when that package is installed (reference: src/offload_adam/_pretrained.py:18-114).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import List, Union

import torch

from .qweight.base import QWeightBase


def _directory_shards(directory: Path) -> List[Path]:
    index = directory / "model.safetensors.index.json"
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
        return [directory / name for name in sorted(set(weight_map.values()))]
    single = directory / "model.safetensors"
    if single.exists():
        return [single]
    anything = sorted(directory.glob("*.safetensors"))
    if not anything:
        raise FileNotFoundError(
            f"No safetensors files under {directory} (looked for model.safetensors, "
            f"model.safetensors.index.json, or any *.safetensors)."
        )
    return anything


def resolve_safetensors_paths(pretrained_name_or_path: Union[str, Path]) -> List[Path]:
    """Local safetensors files behind a ``from_pretrained`` identifier."""
    here = Path(pretrained_name_or_path)
    if here.is_file():
        return [here]
    if here.is_dir():
        return _directory_shards(here)
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise ImportError(
            f"'{pretrained_name_or_path}' is not a local file or directory and "
            "`huggingface_hub` is not installed. Install it or pass a local path."
        ) from e
    local = snapshot_download(
        repo_id=str(pretrained_name_or_path),
        allow_patterns=["*.safetensors", "*.safetensors.index.json"],
    )
    return _directory_shards(Path(local))


@torch.no_grad()
def stream_master_from_pretrained(optim, pretrained_name_or_path, model, *, strict: bool) -> List[str]:
    """Copy each quantized param's checkpoint tensor into its fp32 master.

    Only one tensor is resident at a time.  Non-quantized params are skipped:
    their master was widened losslessly from the live weights at optimizer
    construction.  Returns the sorted names of quantized params that no file
    contained; ``strict=True`` turns a non-empty list into ``ValueError``.
    """
    from safetensors import safe_open

    by_name = {n: p for n, p in model.named_parameters() if p.requires_grad}
    wanted = {n for n, p in by_name.items() if isinstance(p.data, QWeightBase)}
    init = getattr(optim, "_init_state_if_empty", None)
    done = set()
    for path in resolve_safetensors_paths(pretrained_name_or_path):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for key in wanted.intersection(f.keys()):
                p = by_name[key]
                st = optim.state[p]
                if init is not None:
                    init(p, st)
                if "master_params" not in st:
                    continue
                optim._copy_master(p, f.get_tensor(key))
                if "master_filled" in st:
                    st["master_filled"] = True
                done.add(key)
    missing = sorted(wanted - done)
    if strict and missing:
        raise ValueError(
            f"load_master_from_pretrained(strict=True): {len(missing)} quant param(s) "
            f"have no matching key in the checkpoint: {missing}"
        )
    return missing
