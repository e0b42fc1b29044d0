"""Multi-GPU training with ``DistributedOffloadAdam`` (ZeRO-1), one rank per GPU.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 \
        examples/multi_gpu/train.py --model-name llama3-8b --tokens-per-sample 4096 \
        --grad-accum-steps 4 --max-grad-norm 1.0

Every rank holds the full bf16 model and runs its own micro-batches; the optimizer
averages gradients, updates its row shard of every large tensor and refreshes all
replicas itself (do not wrap the model in DDP).  ``--comm symm`` (default on NVLink
machines) uses this package's peer-memory kernels, ``--comm nccl`` the collectives of
``torch.distributed`` (reference: examples/multi_gpu/train.py).
"""

import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import common  # noqa: E402
from offload_adam_b200 import DistributedOffloadAdam  # noqa: E402


def main():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    common.add_common_args(p)
    p.add_argument("--per-rank-batch-size", type=int, default=1)
    p.add_argument("--comm", choices=["auto", "symm", "nccl"], default="auto")
    p.add_argument("--grad-layout", choices=["full", "shard"], default="full",
                   help="'shard': reduce-scatter every micro-batch and accumulate only this rank's rows "
                        "(gradient memory divided by the world size; what a 70B model needs)")
    args = p.parse_args()
    common.validate(args)
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(args.seed)
    torch.backends.cuda.matmul.allow_tf32 = True
    model = common.build_model(args, device)
    opt = DistributedOffloadAdam(
        model, lr=args.lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=args.weight_decay, mode=args.mode,
        decoupled_weight_decay=True, max_grad_norm=args.max_grad_norm, numa_node=common.numa_arg(args.numa_node),
        prefetch_policy=args.prefetch_policy, verbose=1, transfer=args.transfer,
        grad_residency=args.grad_residency, comm=args.comm, seed=args.seed,
        staging_bytes=common.staging_arg(args), grad_layout=args.grad_layout)
    if rank == 0:
        print(f"model={args.model_name} world_size={world} device={torch.cuda.get_device_name(local_rank)} "
              f"mode={args.mode} comm={opt.comm}", flush=True)

    def mean_loss(t):
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        return t

    summary = common.train(args, model, opt, args.per_rank_batch_size, device, world=world, rank=rank,
                           reduce_loss=mean_loss, barrier=dist.barrier)
    if rank == 0:
        summary["comm"] = opt.comm
        common.emit(args, summary)
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except KeyboardInterrupt:
        sys.exit(130)
