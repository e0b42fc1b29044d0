"""Quantization-aware training: weight-only fake quantization of every linear layer
(int4 / int8 / NF4 / NVFP4) on top of ``OffloadAdam`` or ``Adam``.

    python examples/qat/train.py --quant nvfp4 --tokens-per-sample 2048 --batch-size 2

The optimizer keeps an fp32 master of each quantized weight (``mode=fp32_master`` is
required) and re-quantizes the packed weight from it after every step.  Pass
``--load-master-from <safetensors file | directory | hub id>`` to refill the master
losslessly from the checkpoint the model was quantized from; ``--save-dir`` writes a
plain-tensor safetensors checkpoint plus the matching HF ``quantization_config``.
With ``--hf-model <checkpoint>`` a HuggingFace causal LM is trained, the master is
refilled from that same checkpoint unless ``--load-master-from`` names another, and the
export goes through ``save_quantized_pretrained`` (loadable by HF / vLLM)
(reference: examples/qat/train.py).
"""

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import common  # noqa: E402
from offload_adam_b200 import Adam, OffloadAdam  # noqa: E402
from offload_adam_b200.qweight import (Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight,  # noqa: E402
                                       quantize_linears, save_quantized_pretrained)

QUANT = {"none": None, "int4": Int4QWeight, "int8": Int8QWeight, "nf4": NF4QWeight, "nvfp4": NVFP4QWeight}


def main():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    common.add_common_args(p)
    p.add_argument("--enable-offloading", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--quant", choices=list(QUANT), default="none")
    p.add_argument("--quant-group-size", type=int, default=128, help="int4 group size")
    p.add_argument("--quant-blocksize", type=int, default=64, help="NF4 block size")
    p.add_argument("--quant-skip-patterns", nargs="+", default=["lm_head"])
    p.add_argument("--load-master-from", default=None)
    p.add_argument("--save-dir", type=Path, default=None)
    args = p.parse_args()
    common.validate(args)
    if args.quant != "none" and args.mode != "fp32_master":
        raise ValueError(f"--quant {args.quant!r} requires --mode fp32_master; got {args.mode!r}")
    torch.manual_seed(args.seed)
    torch.backends.cuda.matmul.allow_tf32 = True
    device = torch.device("cuda", 0)
    model = common.build_model(args, device)
    cls = QUANT[args.quant]
    kw = {}
    if cls is not None:
        if args.quant == "int4":
            kw["group_size"] = args.quant_group_size
        elif args.quant == "nf4":
            kw["blocksize"] = args.quant_blocksize
        rep = quantize_linears(model, cls, skip_patterns=tuple(args.quant_skip_patterns), **kw)
        print(f"quantization={args.quant} kwargs={kw} quantized={len(rep.quantized)} "
              f"excluded={len(rep.excluded)} incompatible={len(rep.incompatible)}", flush=True)
    hp = dict(lr=args.lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=args.weight_decay, mode=args.mode,
              decoupled_weight_decay=True)
    if args.enable_offloading:
        opt = OffloadAdam(model, numa_node=common.numa_arg(args.numa_node), verbose=1,
                          max_grad_norm=args.max_grad_norm, prefetch_policy=args.prefetch_policy,
                          transfer=args.transfer, grad_residency=args.grad_residency,
                          staging_bytes=common.staging_arg(args), **hp)
    else:
        opt = Adam(model.parameters(), **hp)
    hf = getattr(model, "hf", None)  # the HuggingFace module when --hf-model is given
    master_from = args.load_master_from
    if master_from is None and hf is not None and common.has_weights(args.hf_model):
        master_from = args.hf_model  # the checkpoint from_pretrained just read
    if master_from and cls is not None:
        missing = opt.load_master_from_pretrained(master_from, hf if hf is not None else model)
        print(f"master refilled from {master_from}; unmatched: {len(missing)}", flush=True)
    summary = common.train(args, model, opt, args.batch_size, device)
    summary.update(quant=args.quant, quant_group_size=args.quant_group_size,
                   quant_skip_patterns=args.quant_skip_patterns, enable_offloading=args.enable_offloading)
    common.emit(args, summary)
    if args.save_dir is not None and hf is not None:
        if hasattr(opt, "synchronize"):
            opt.synchronize()
        if cls is not None:
            save_quantized_pretrained(hf, args.save_dir, cls, skip_patterns=tuple(args.quant_skip_patterns), **kw)
        else:
            hf.save_pretrained(args.save_dir)
    elif args.save_dir is not None:
        from safetensors.torch import save_file
        args.save_dir.mkdir(parents=True, exist_ok=True)
        save_file({k: v.contiguous() for k, v in model.state_dict().items()}, str(args.save_dir / "model.safetensors"))
        cfg = {"model_type": "llama"}
        if cls is not None:
            cfg["quantization_config"] = cls.build_hf_quantization_config(
                skip_patterns=tuple(args.quant_skip_patterns), **kw)
        (args.save_dir / "config.json").write_text(json.dumps(cfg, indent=2))


if __name__ == "__main__":
    try:
        main()
    except KeyboardInterrupt:
        sys.exit(130)
