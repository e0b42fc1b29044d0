"""Peer-memory kernels over NVLink, timed on real peers (2 to 8 GPUs, one process each).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m offload_adam_b200.utils.nvlink_bench --elems 67108864
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m offload_adam_b200.utils.nvlink_bench --kernel-list

Cases (every rank runs the same launch at the same time, as in a training step; times are
CUDA events on the launching stream, max over ranks):

``peer_pull``      one neighbour's buffer read with this package's plain 256-bit peer loads and
                   written to local memory (no library copy touches peer memory): the link
                   rate these kernels can reach; fractions are quoted against ``--link-gbs``
                   (default 770 GB/s per direction, the peer-copy rate measured on this kind
                   of node) and this figure is printed beside them
``pull_normsq``    rows pulled from all replicas, averaged, squared norm (clip path, backward side)
``adam_push``      Adam on the shard, new bf16 rows stored into all replicas (clip path, step side)
``pull_adam_push`` both in one pass (no-clip path)
``adam_quant_push`` Adam on the fp32 master, re-quantize, packed rows stored into all replicas

For each case the bytes that must cross NVLink per rank and the achieved fraction of the
reference link rate are printed as one JSON line by rank 0.  Buffers are symmetric
allocations of ``torch.distributed._symmetric_memory`` bound without multicast; all loads
and stores are plain peer accesses.

``--kernel-list`` instead trains a small model for a few steps with ``DistributedOffloadAdam``
on the peer-memory path under ``torch.profiler`` and prints the names of all GPU kernels
that ran between the end of the last backward pass and the end of ``step()``, so that the
absence of NCCL kernels on that path can be read off.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _events_ms(fn, iters, warmup=2):
    for _ in range(warmup):
        dist.barrier()
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best = min(best, t.item())
    return best


def _symm_buffer(nbytes, group):
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(nbytes, dtype=torch.uint8, device="cuda")
    t.zero_()
    h = symm_mem.rendezvous(t, group)
    return t, [int(p) for p in h.buffer_ptrs], h


def run_cases(args):
    from .. import _ext
    from ..ops import grad_ops
    from ..ops.oracle import beta_hat
    C = _ext.load(required=True)
    rank, world = dist.get_rank(), dist.get_world_size()
    group = dist.group.WORLD
    n = args.elems // world * world
    shard = n // world
    out = []

    grads, gptrs, hg = _symm_buffer(n * 2, group)
    params, pptrs, hp = _symm_buffer(n * 2, group)
    grads.view(torch.bfloat16).copy_((torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16))
    torch.cuda.synchronize()
    dist.barrier()

    # ---- the link itself: pull a neighbour's whole buffer with plain peer loads
    peer = (rank + 1) % world
    local = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    t = _events_ms(lambda: C.peer_reduce(local, [gptrs[peer]], 1.0, None, None, None, 0, 0), args.iters)
    link = float(args.link_gbs)
    out.append({"case": "peer_pull", "bytes": n * 2, "ms": t, "GBs": n * 2 / t / 1e6, "link_GBs_reference": link})

    red = torch.empty(shard, dtype=torch.bfloat16, device="cuda")
    sq = torch.zeros(1, device="cuda")
    scratch = grad_ops.sumsq_scratch("cuda")
    my_g = [b + rank * shard * 2 for b in gptrs]
    my_p = [b + rank * shard * 2 for b in pptrs]
    remote = (world - 1) * shard * 2  # bytes over NVLink per rank, one direction

    t = _events_ms(lambda: C.peer_reduce(red, my_g, 1.0 / world, sq, scratch, None, 0, 0), args.iters)
    out.append({"case": "pull_normsq", "nvlink_bytes_in": remote, "ms": t, "GBs_in": remote / t / 1e6,
                "fraction_of_link_reference": remote / t / 1e6 / link})

    m = torch.zeros(shard, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros(shard, dtype=torch.bfloat16, device="cuda")
    master = torch.randn(shard, device="cuda") * 0.02
    step = [1]

    def adam(g, g_peers, p_peers):
        step[0] += 1
        C.adam_step(1, None, g, None, m, v, master, 1e-4, 0.01, beta_hat(0.9, step[0]), beta_hat(0.999, step[0]),
                    1e-8, True, None, 0, 0, None, 0, 0, g_peers, 1.0 / world, p_peers, None)

    t = _events_ms(lambda: adam(red, [], my_p), args.iters)
    hbm = shard * 18 / t / 1e6
    out.append({"case": "adam_push", "nvlink_bytes_out": remote, "ms": t, "GBs_out": remote / t / 1e6,
                "fraction_of_link_reference": remote / t / 1e6 / link, "local_hbm_GBs": hbm})
    t = _events_ms(lambda: adam(None, my_g, my_p), args.iters)
    # every rank runs the same launch: a rank's inbound link carries the gradients it pulls AND
    # the parameters the others push into it (outbound: what it serves and what it pushes)
    out.append({"case": "pull_adam_push", "nvlink_bytes_in": 2 * remote, "nvlink_bytes_out": 2 * remote, "ms": t,
                "GBs_each_direction": 2 * remote / t / 1e6,
                "fraction_of_link_reference": 2 * remote / t / 1e6 / link})

    # ---- quantized weight: rows x cols, this rank owns rows/world of them
    cols = args.cols
    rows = (n // cols) // (32 * world) * (32 * world)
    if rows > 0:
        my_rows = rows // world
        qn = my_rows * cols
        for fmt, fid, group_sz, b0, b1 in (
                ("nf4", C.QFMT_NF4, 64, rows * cols // 2, rows * cols // 64 * 4),
                ("int4", C.QFMT_INT4, 128, rows * cols // 2, rows * cols // 128 * 2),
                ("int8", C.QFMT_INT8, 0, rows * cols, rows * 2)):
            p0, p0ptrs, _ = _symm_buffer(b0, group)
            p1, p1ptrs, _ = _symm_buffer(max(b1, 256), group)
            spec = C.QuantSpec(fid, rows, cols, rank * my_rows, group_sz, C.QDT_BF16, p0ptrs, p1ptrs)
            qm, qv = m[:qn].view(my_rows, cols), v[:qn].view(my_rows, cols)
            qmaster, qg = master[:qn].view(my_rows, cols), red[:qn].view(my_rows, cols)

            def fused():
                step[0] += 1
                C.adam_quant_push(spec, qg, None, qm, qv, qmaster, 1e-4, 0.01, beta_hat(0.9, step[0]),
                                  beta_hat(0.999, step[0]), 1e-8, True, None, 0, 0, [], 1.0, None)

            t = _events_ms(fused, args.iters)
            wire = (world - 1) * (b0 + b1) // world
            out.append({"case": "adam_quant_push", "format": fmt, "rows": rows, "cols": cols, "ms": t,
                        "nvlink_bytes_out": wire, "GBs_out": wire / t / 1e6,
                        "fraction_of_link_reference": wire / t / 1e6 / link,
                        "local_hbm_GBs": qn * 18 / t / 1e6,
                        "fp32_gather_bytes_of_the_reference": (world - 1) * qn * 4})
            del p0, p1
    if rank == 0:
        for row in out:
            row["world"] = world
            print(json.dumps(row), flush=True)


def kernel_list(args):
    """Kernel names of the optimizer step on the peer-memory path, from torch.profiler."""
    import torch.nn as nn
    from torch.profiler import ProfilerActivity, profile, record_function

    from .. import DistributedOffloadAdam
    rank = dist.get_rank()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(512, 2048, bias=False), nn.ReLU(), nn.Linear(2048, 512, bias=False),
                          nn.ReLU(), nn.Linear(512, 64, bias=True)).to(torch.bfloat16).cuda()
    opt = DistributedOffloadAdam(model, lr=1e-3, mode="fp32_master", max_grad_norm=(args.clip if args.clip > 0 else None), comm="symm",
                                 decoupled_weight_decay=True, inplace_param_threshold=4096, chunk_elems=1 << 16)
    assert opt.comm == "symm"
    x = torch.randn(64, 512, device="cuda").to(torch.bfloat16)

    def one_step(tag=False):
        for micro in range(2):
            opt.ready_for_optimizer_step = micro == 1
            model(x).float().pow(2).mean().backward()
        if tag:
            with record_function("oab_step_region"):
                opt.step()
                torch.cuda.synchronize()
        else:
            opt.step()

    for _ in range(3):
        one_step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        one_step(tag=True)
    opt.synchronize()
    events = prof.events()
    region = [e for e in events if e.name == "oab_step_region"]
    names = {}
    if region:
        t0, t1 = region[0].time_range.start, region[0].time_range.end
        for e in events:
            if e.device_type is not None and str(e.device_type).endswith("CUDA") and t0 <= e.time_range.start <= t1:
                names[e.name] = names.get(e.name, 0) + 1
    all_kernels = {}
    for e in events:
        if e.device_type is not None and str(e.device_type).endswith("CUDA"):
            all_kernels[e.name] = all_kernels.get(e.name, 0) + 1
    if rank == 0:
        print(json.dumps({"case": "kernel_list", "clip": args.clip, "world": dist.get_world_size(),
                          "kernels_in_step": names,
                          "nccl_kernels_in_step": sorted(k for k in names if "nccl" in k.lower()),
                          "nccl_kernels_in_whole_iteration": sorted(k for k in all_kernels if "nccl" in k.lower())}),
              flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--elems", type=int, default=64 << 20, help="elements of the whole tensor (all ranks)")
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--link-gbs", type=float, default=770.0,
                    help="peer-copy rate per direction that fractions are quoted against")
    ap.add_argument("--kernel-list", action="store_true")
    ap.add_argument("--clip", type=float, default=1.0, help="--kernel-list: clipping threshold, 0 for the step-in-backward path")
    args = ap.parse_args()
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    try:
        if args.kernel_list:
            kernel_list(args)
        else:
            run_cases(args)
    finally:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
