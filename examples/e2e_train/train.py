"""End-to-end training on synthetic tokens with ``OffloadAdam`` or the on-GPU ``Adam``.

    python examples/e2e_train/train.py --model-name llama3-8b --mode fp32_master \
        --tokens-per-sample 4096 --grad-accum-steps 4 --max-grad-norm 1.0

Builds the Llama-style model of this package with random weights, feeds it uniform
random token batches and reports per-step timing, tokens/s, peak GPU memory and a JSON
summary (reference: examples/e2e_train/train.py).
"""

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import common  # noqa: E402
from offload_adam_b200 import Adam, OffloadAdam  # noqa: E402


def main():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    common.add_common_args(p)
    p.add_argument("--enable-offloading", action=argparse.BooleanOptionalAction, default=True,
                   help="OffloadAdam when enabled, plain Adam otherwise")
    p.add_argument("--batch-size", type=int, default=1)
    args = p.parse_args()
    common.validate(args)
    torch.manual_seed(args.seed)
    torch.backends.cuda.matmul.allow_tf32 = True
    device = torch.device("cuda", 0)
    model = common.build_model(args, device)
    hp = dict(lr=args.lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=args.weight_decay, mode=args.mode,
              decoupled_weight_decay=True)
    if args.enable_offloading:
        opt = OffloadAdam(model, numa_node=common.numa_arg(args.numa_node), verbose=1,
                          max_grad_norm=args.max_grad_norm, prefetch_policy=args.prefetch_policy,
                          transfer=args.transfer, grad_residency=args.grad_residency,
                          staging_bytes=common.staging_arg(args), **hp)
    else:
        opt = Adam(model.parameters(), **hp)
    print(f"model={args.model_name} device={torch.cuda.get_device_name(0)} "
          f"enable_offloading={args.enable_offloading} mode={args.mode}", flush=True)
    summary = common.train(args, model, opt, args.batch_size, device)
    summary["enable_offloading"] = args.enable_offloading
    common.emit(args, summary)


if __name__ == "__main__":
    try:
        main()
    except KeyboardInterrupt:
        sys.exit(130)
