"""Pieces shared by the example trainers: model construction, synthetic batches, the
timed training loop and the JSON summary (reference: examples/e2e_train/train.py:106-233)."""

from __future__ import annotations

import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from offload_adam_b200.models.hf import causal_lm_loss  # noqa: E402
from offload_adam_b200.models.llama import (build_llama, llama3_8b, llama3_70b,  # noqa: E402
                                            qwen3_8b, tiny_llama)

MODELS = {"llama3-8b": llama3_8b, "llama3-70b": llama3_70b, "qwen3-8b": qwen3_8b, "tiny": tiny_llama}
MODES = ["stochastic_rounding", "fp32_master", "fp31_master", "fp32_master_custom_rounding"]


def add_common_args(p):
    p.add_argument("--model-name", default="llama3-8b", choices=list(MODELS))
    p.add_argument("--hf-model", default=None,
                   help="train a HuggingFace causal LM instead of the package's own Llama: a local checkpoint "
                        "directory or hub id (weights are loaded with AutoModelForCausalLM.from_pretrained), or "
                        "a directory / file holding only a config.json (random-init weights of that architecture)")
    p.add_argument("--full-logits", action="store_true",
                   help="with --hf-model: use the module's own loss (full fp32 logits) instead of the chunked "
                        "linear cross-entropy that never materialises them")
    p.add_argument("--liger-fused-linear-ce", action="store_true",
                   help="accepted so that the reference trainers' command lines keep working; the chunked linear "
                        "cross-entropy is the default here and needs no extra package")
    p.add_argument("--layers", type=int, default=None, help="override the number of layers")
    p.add_argument("--mode", choices=MODES, default="fp32_master")
    p.add_argument("--tokens-per-sample", type=int, default=2048)
    p.add_argument("--grad-accum-steps", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup-steps", type=int, default=2)
    p.add_argument("--lr", type=float, default=1e-4)
    p.add_argument("--weight-decay", type=float, default=0.01)
    p.add_argument("--max-grad-norm", type=float, default=None,
                   help="L2 global-norm clipping; selects the one-shot .step() path")
    p.add_argument("--numa-node", default="auto", help="'auto', a node id, or 'none'")
    p.add_argument("--prefetch-policy", choices=["eager", "lazy"], default="eager")
    p.add_argument("--transfer", choices=["auto", "staged", "zero_copy"], default="auto")
    p.add_argument("--grad-residency", choices=["auto", "host", "device"], default="auto")
    p.add_argument("--staging-gib", type=float, default=None,
                   help="device staging buffer of the offloaded optimizers in GiB (default: the state "
                        "size, at most a quarter of the GPU); smaller saves memory, larger hides more PCIe time")
    p.add_argument("--gradient-checkpointing", action="store_true")
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--json-output", type=Path)


def staging_arg(args):
    return None if args.staging_gib is None else int(args.staging_gib * 2**30)


def numa_arg(v):
    return None if v == "none" else (v if v == "auto" else int(v))


def validate(args):
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is required.")
    for name in ("tokens_per_sample", "grad_accum_steps", "steps"):
        if getattr(args, name) < 1:
            raise ValueError(f"--{name.replace('_', '-')} must be >= 1")
    if not 0 <= args.warmup_steps < args.steps:
        raise ValueError("--warmup-steps must be in [0, --steps)")


class _HFCausalLM(torch.nn.Module):
    """Gives a HuggingFace causal LM the call signature the example loop uses
    (``model(ids, labels=ids)`` returns the loss) and keeps ``.config`` reachable.  The
    head and the loss run chunk by chunk (``offload_adam_b200.models.hf.causal_lm_loss``)
    unless ``full_logits`` asks for the module's own loss."""

    def __init__(self, hf, full_logits=False):
        super().__init__()
        self.hf = hf
        self.config = hf.config
        self.full_logits = full_logits

    def forward(self, ids, labels=None):
        if self.full_logits or labels is None:
            return self.hf(input_ids=ids, labels=labels).loss
        return causal_lm_loss(self.hf, ids, labels)

    def gradient_checkpointing_enable(self):
        self.hf.gradient_checkpointing_enable()

    def save_pretrained(self, *a, **kw):
        return self.hf.save_pretrained(*a, **kw)


def has_weights(src):
    """False when ``src`` is a bare config (file, or directory without weight files)."""
    import os
    if os.path.isfile(src):
        return False
    if os.path.isdir(src):
        return any(f.endswith((".safetensors", ".bin")) for f in os.listdir(src))
    return True  # a hub id


def build_hf_model(args, device):
    """``--hf-model``: pretrained weights when the path or id has any, else random
    initialisation from its config (reference: examples/e2e_train/train.py:117-129)."""
    from transformers import AutoConfig, AutoModelForCausalLM
    src = args.hf_model
    if not has_weights(src):
        cfg = AutoConfig.from_pretrained(src)
        if args.layers is not None:
            cfg.num_hidden_layers = args.layers
        cfg.use_cache = False
        torch.manual_seed(args.seed)
        hf = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16, attn_implementation="sdpa")
    else:
        hf = AutoModelForCausalLM.from_pretrained(src, dtype=torch.bfloat16, attn_implementation="sdpa")
        hf.config.use_cache = False
    model = _HFCausalLM(hf.to(torch.bfloat16).to(device), full_logits=getattr(args, "full_logits", False))
    model.train()
    if args.gradient_checkpointing:
        model.gradient_checkpointing_enable()
    return model


def build_model(args, device):
    if getattr(args, "hf_model", None):
        return build_hf_model(args, device)
    cfg = MODELS[args.model_name]()
    if args.layers is not None:
        cfg.num_layers = args.layers
    model = build_llama(cfg, device=device, dtype=torch.bfloat16, seed=args.seed)
    model.train()
    if args.gradient_checkpointing:
        model.gradient_checkpointing_enable()
    return model


def batches(args, vocab, device, batch_size, seed):
    gen = torch.Generator(device=device).manual_seed(seed)
    while True:
        yield torch.randint(0, vocab, (batch_size, args.tokens_per_sample), device=device, generator=gen)


def train(args, model, optimizer, batch_size, device, world=1, rank=0, reduce_loss=None, barrier=None):
    """Synthetic-token training loop; prints one line per step and returns the summary."""
    vocab = model.config.vocab_size
    it = batches(args, vocab, device, batch_size, args.seed + rank)
    tokens_per_step = batch_size * args.tokens_per_sample * args.grad_accum_steps * world
    times, losses = [], []
    torch.cuda.reset_peak_memory_stats()
    for step in range(args.steps):
        optimizer.zero_grad(set_to_none=True)
        torch.cuda.synchronize()
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for micro in range(args.grad_accum_steps):
            if hasattr(optimizer, "ready_for_optimizer_step"):
                optimizer.ready_for_optimizer_step = micro == args.grad_accum_steps - 1
            ids = next(it)
            loss = model(ids, labels=ids)
            (loss / args.grad_accum_steps).backward()
        optimizer.step()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        dt = time.perf_counter() - t0
        value = loss.detach().float()
        if reduce_loss:
            value = reduce_loss(value)
        value = value.item()
        phase = "warmup" if step < args.warmup_steps else "measure"
        if rank == 0:
            print(f"step={step + 1}/{args.steps} phase={phase} loss={value:.4f} step_time_s={dt:.4f} "
                  f"tokens_per_s={tokens_per_step / dt:.1f} "
                  f"cuda_peak_gb={torch.cuda.max_memory_allocated() / 1024**3:.2f}", flush=True)
        if step >= args.warmup_steps:
            times.append(dt)
            losses.append(value)
    return {
        "model_name": args.model_name, "mode": args.mode, "world_size": world,
        "batch_size": batch_size, "tokens_per_sample": args.tokens_per_sample,
        "grad_accum_steps": args.grad_accum_steps, "effective_batch_tokens": tokens_per_step,
        "gradient_checkpointing": args.gradient_checkpointing, "measured_steps": len(times),
        "warmup_steps": args.warmup_steps, "avg_loss": sum(losses) / len(losses),
        "avg_step_time_s": sum(times) / len(times),
        "tokens_per_second": tokens_per_step * len(times) / sum(times),
        "max_cuda_memory_gb": torch.cuda.max_memory_allocated() / 1024**3,
    }


def emit(args, summary):
    print(json.dumps(summary, indent=2, sort_keys=True))
    if args.json_output is not None:
        args.json_output.parent.mkdir(parents=True, exist_ok=True)
        args.json_output.write_text(json.dumps(summary, indent=2, sort_keys=True) + "\n", encoding="utf-8")
