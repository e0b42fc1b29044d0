#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B-shaped full-parameter training with host-offloaded Adam.

    python bench.py --gpus 1 --steps K --warmup W                 # this framework
    python bench.py --impl reference --gpus 1 --steps K --warmup W  # unmodified reference

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...`` (one rank per GPU).

Metric: training tokens/s of the whole job (all ranks), Llama-3-8B shape, synthetic
uniform tokens, random-init bf16 weights, ``DistributedOffloadAdam`` ZeRO-1,
mode=fp32_master, max_grad_norm=1.0, AdamW wd 0.01, lr 1e-4, per-rank micro-batch
1 x 4096, 4 accumulation micro-batches per optimizer step.  ``--preset single`` selects
the single-GPU stochastic-rounding configuration (OffloadAdam, no clipping, 8
micro-batches).  Rank 0 prints one JSON line.

Timing: W untimed warm-up steps, then exactly K steps between a barrier +
``torch.cuda.synchronize()`` on both sides, measured with CUDA events on the main
stream, max over ranks.  The closing event is recorded after every stream of the
process has drained, so the write-back of the last step's optimizer state to the host
is inside the timed region (in a longer run it overlaps the next forward pass).  The
working set (16 GB of parameters plus activations) is far larger than L2, so no explicit
L2 flush is needed between iterations.  ``value`` is the device-timed number with inputs
already on the GPU; ``e2e`` repeats the measurement through the public API with every
micro-batch's token ids copied from pinned host memory and the step's loss read back to
the host.

``--model-impl hf`` trains the same HuggingFace ``LlamaForCausalLM`` the reference arm
uses (full fp32 logits) with this package's optimizer instead of the package's own
Llama (chunked linear cross-entropy): the pair of runs separates the optimizer's share
of a speed-up from the model code's.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))

PRESETS = {
    # BASELINE config 3: ZeRO-1 fp32_master + clipping at 1/2/4/8 GPUs
    "zero1": dict(optimizer="distributed", mode="fp32_master", max_grad_norm=1.0, ga=4,
                  weight_decay=0.01, lr=1e-4, seq=4096, mb=1),
    # BASELINE config 2: single-GPU stochastic rounding, step inside backward
    "single": dict(optimizer="offload", mode="stochastic_rounding", max_grad_norm=None, ga=8,
                   weight_decay=0.01, lr=1e-4, seq=4096, mb=1),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--preset", choices=list(PRESETS), default="zero1")
    ap.add_argument("--model", choices=["llama3-8b", "llama3-70b", "tiny"], default="llama3-8b")
    ap.add_argument("--model-impl", choices=["own", "hf"], default="own",
                    help="this framework's arm: the package's Llama, or the HuggingFace module the reference arm trains")
    ap.add_argument("--hf-chunked-loss", action="store_true",
                    help="with --model-impl hf: head and loss chunk by chunk (models.hf.causal_lm_loss) instead "
                         "of the module's own full-logits loss")
    ap.add_argument("--no-resident", action="store_true", help="stream all optimizer state every step")
    ap.add_argument("--resident-writeback", default="step", choices=["step", "on_demand"],
                    help="'on_demand': resident state is copied to the host only when the host copy is "
                         "asked for (here: once, at the end of the timed region); not the default")
    ap.add_argument("--symmetric-model", action="store_true",
                    help="create the large parameters directly in symmetric memory (default for llama3-70b with "
                         "more than one GPU: a second copy of the weights would not fit)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: override layer count")
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--ga", type=int, default=None)
    ap.add_argument("--mb", type=int, default=None, help="micro-batch size per rank")
    ap.add_argument("--quant", choices=["none", "nvfp4", "nf4", "int4", "int8"], default="none",
                    help="QAT: weight-only quantized linear layers (lm_head stays dense); needs mode fp32_master")
    ap.add_argument("--mode", default=None)
    ap.add_argument("--transfer", default="auto")
    ap.add_argument("--grad-residency", default="auto")
    ap.add_argument("--comm", default="auto", help="distributed path: auto | symm | nccl")
    ap.add_argument("--grad-layout", default="full", choices=["full", "shard"],
                    help="distributed: 'shard' reduce-scatters every micro-batch (70B memory plan)")
    ap.add_argument("--max-ctas", type=int, default=0)
    ap.add_argument("--staging-gib", type=float, default=None, help="size of the staging ring (default: optimizer default)")
    ap.add_argument("--prefetch-inflight", type=int, default=None,
                    help="early-H2D chunks in the copy engine at once (0: unbounded)")
    ap.add_argument("--chunk-elems", type=int, default=None)
    ap.add_argument("--sync-writeback", action="store_true", help="issue D2H write-backs inline")
    ap.add_argument("--grad-ckpt", action="store_true", help="activation checkpointing per layer")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--profile-range", action="store_true",
                    help="after the timed region, run one more step between cudaProfilerStart/Stop "
                         "(for `ncu --profile-from-start off`); not part of any reported number")
    ap.add_argument("--verbose", type=int, default=0)
    return ap.parse_args()


# --------------------------------------------------------------------------- utils
def setup_dist(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if "MASTER_ADDR" not in os.environ:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
    if "MASTER_PORT" not in os.environ:
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        s.close()
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", local_rank))
    return rank, local_rank, world


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during a region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.strip().split(",") for r in open(self.path) if r.strip()]
            os.unlink(self.path)
        except Exception:
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


def max_over_ranks(x, device):
    t = torch.tensor([float(x)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def host_memory_shortfall(args, preset, world):
    """None when the pinned host memory the run needs fits in what the machine has free,
    else a one-line reason.  Per parameter element and rank: optimizer state / world (8 B
    in fp32_master, 4 B with stochastic rounding, 6 B otherwise) plus, for the reference,
    a full-shape bf16 gradient buffer on every rank (its host gradients are never sharded)."""
    d = model_dims(args)
    layer = 2 * d.hidden_size * (d.num_heads + d.num_kv_heads) * d.head_dim + 3 * d.hidden_size * d.intermediate_size
    n = d.num_layers * layer + d.vocab_size * d.hidden_size * (1 if d.tie_embeddings else 2)
    state = {"fp32_master": 8, "stochastic_rounding": 4}.get(preset["mode"], 6)
    sharded = preset["optimizer"] == "distributed"
    per_rank = n * state / (world if sharded else 1)
    if args.impl == "reference":
        per_rank += 2 * n
    elif args.grad_residency == "host":
        per_rank += 2 * n / (world if args.grad_layout == "shard" else 1)
    need = per_rank * world
    try:
        avail = next(int(line.split()[1]) * 1024 for line in open("/proc/meminfo") if line.startswith("MemAvailable"))
    except Exception:
        return None
    if need > 0.9 * avail:
        return (f"needs {need / 2**30:.0f} GiB of pinned host memory on this node ({per_rank / 2**30:.0f} GiB per rank x "
                f"{world}) but only {avail / 2**30:.0f} GiB are available")
    return None


# ------------------------------------------------------------------ model builders
def model_dims(args):
    from offload_adam_b200.models.llama import llama3_8b, llama3_70b, tiny_llama
    cfg = {"llama3-8b": llama3_8b, "llama3-70b": llama3_70b, "tiny": tiny_llama}[args.model]()
    if args.layers is not None:
        cfg.num_layers = args.layers
    return cfg


def build_ours(args, preset, device):
    from offload_adam_b200 import DistributedOffloadAdam, OffloadAdam
    from offload_adam_b200.models.llama import build_llama
    cfg = model_dims(args)
    if args.model_impl == "hf":
        model, _ = build_hf_llama(args, preset, device)
    else:
        symmetric = (args.symmetric_model or args.model == "llama3-70b") and dist.get_world_size() > 1 \
            and args.comm != "nccl"
        model = build_llama(cfg, device=device, dtype=torch.bfloat16, seed=0,
                            symmetric_group=dist.group.WORLD if symmetric else None)
        model.train()
        if args.grad_ckpt:
            model.gradient_checkpointing_enable()
    if args.quant != "none":
        from offload_adam_b200 import qweight
        cls = {"nvfp4": qweight.NVFP4QWeight, "nf4": qweight.NF4QWeight, "int4": qweight.Int4QWeight,
               "int8": qweight.Int8QWeight}[args.quant]
        qweight.quantize_linears(model, cls, skip_patterns=("lm_head",))
    common = dict(lr=preset["lr"], betas=(0.9, 0.999), eps=1e-8, weight_decay=preset["weight_decay"],
                  mode=preset["mode"], decoupled_weight_decay=True, max_grad_norm=preset["max_grad_norm"],
                  verbose=args.verbose, transfer=args.transfer, grad_residency=args.grad_residency,
                  max_ctas=args.max_ctas, seed=1234)
    if args.staging_gib is not None:
        common["staging_bytes"] = int(args.staging_gib * 2**30)
    if args.chunk_elems is not None:
        common["chunk_elems"] = args.chunk_elems
    if args.sync_writeback:
        common["async_writeback"] = False
    if args.prefetch_inflight is not None:
        common["prefetch_inflight"] = args.prefetch_inflight
    if args.no_resident:
        common["keep_resident"] = False
    if args.resident_writeback != "step":
        common["resident_writeback"] = args.resident_writeback
    if preset["optimizer"] == "distributed":
        opt = DistributedOffloadAdam(model, comm=args.comm, grad_layout=args.grad_layout, **common)
    else:
        opt = OffloadAdam(model, **common)

    if args.model_impl == "hf" and args.hf_chunked_loss:
        from offload_adam_b200.models.hf import causal_lm_loss

        def loss_fn(ids):
            return causal_lm_loss(model, ids, ids)
    elif args.model_impl == "hf":
        def loss_fn(ids):
            return model(input_ids=ids, labels=ids).loss
    else:
        def loss_fn(ids):
            return model(ids, labels=ids)

    return model, opt, loss_fn, cfg.vocab_size


def build_hf_llama(args, preset, device):
    """Random-init HuggingFace LlamaForCausalLM of the benchmark's shape (bf16, SDPA)."""
    from transformers import LlamaConfig, LlamaForCausalLM
    d = model_dims(args)
    hf = LlamaConfig(vocab_size=d.vocab_size, hidden_size=d.hidden_size, intermediate_size=d.intermediate_size,
                     num_hidden_layers=d.num_layers, num_attention_heads=d.num_heads,
                     num_key_value_heads=d.num_kv_heads, rope_theta=d.rope_theta, rms_norm_eps=d.rms_eps,
                     tie_word_embeddings=d.tie_embeddings, max_position_embeddings=max(8192, preset["seq"]),
                     attn_implementation="sdpa", use_cache=False, initializer_range=0.02)
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(hf)
    finally:
        torch.set_default_dtype(prev)
    model = model.to(torch.bfloat16)
    model.config.use_cache = False
    model.train()
    if args.grad_ckpt:
        model.gradient_checkpointing_enable()
    return model, d.vocab_size


def build_reference(args, preset, device):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import offload_adam as ref  # the unmodified reference package
    model, vocab = build_hf_llama(args, preset, device)
    if args.quant != "none":
        from offload_adam import qweight as rq  # the reference's own formats
        cls = {"nvfp4": rq.NVFP4QWeight, "nf4": rq.NF4QWeight, "int4": rq.Int4QWeight,
               "int8": rq.Int8QWeight}[args.quant]
        rq.quantize_linears(model, cls, skip_patterns=("lm_head",))
    common = dict(lr=preset["lr"], betas=(0.9, 0.999), eps=1e-8, weight_decay=preset["weight_decay"],
                  mode=preset["mode"], decoupled_weight_decay=True, max_grad_norm=preset["max_grad_norm"],
                  verbose=args.verbose)
    if preset["optimizer"] == "distributed":
        opt = ref.DistributedOffloadAdam(model, **common)
    else:
        opt = ref.OffloadAdam(model, **common)

    def loss_fn(ids):
        return model(input_ids=ids, labels=ids).loss

    return model, opt, loss_fn, vocab


# ------------------------------------------------------------------------ training
def run_steps(n_steps, ga, opt, loss_fn, batches_dev=None, batches_host=None, device=None,
              exposed=None, read_loss=lambda t: t.float().item(), host_times=None):
    """One entry of ``batches_*`` per micro-batch (cycled).  With ``batches_host``
    (end-to-end mode) the token ids of a step are copied from pinned host memory at the
    start of that step, on a side stream as a data loader would, and the step's loss is
    read back to the host after its last backward pass."""
    last = None
    k = 0
    copy_stream = torch.cuda.Stream(device) if batches_host is not None else None
    for _ in range(n_steps):
        staged = None
        t_host = [time.perf_counter()]
        if batches_host is not None:
            staged = []
            # no wait for the main stream: like a data loader, the copies may run while the
            # previous step is still executing (the destination tensors are new allocations
            # of the copy stream; the allocator orders their reuse through record_stream)
            with torch.cuda.stream(copy_stream):
                for micro in range(ga):
                    t = batches_host[(k + micro) % len(batches_host)].to(device, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                    staged.append((t, ev))
        for micro in range(ga):
            opt.ready_for_optimizer_step = micro == ga - 1
            if staged is not None:
                ids, ev = staged[micro]
                torch.cuda.current_stream(device).wait_event(ev)
                ids.record_stream(torch.cuda.current_stream(device))
            else:
                ids = batches_dev[k % len(batches_dev)]
            k += 1
            loss = loss_fn(ids)
            (loss / ga).backward()
            last = loss.detach()
        t_host.append(time.perf_counter())  # forward/backward enqueued
        if batches_host is not None:
            # device -> host read of the step's result (4 bytes).  Read where a training
            # script logs it, before the optimizer step is enqueued: the host then waits
            # for the backward pass only and enqueues the step and the next forward
            # while the GPU works, instead of idling until the step has finished.
            last = read_loss(last)
        t_host.append(time.perf_counter())  # loss on the host
        if exposed is not None:
            e0 = torch.cuda.Event(enable_timing=True); e0.record()
        opt.step()
        if exposed is not None:
            e1 = torch.cuda.Event(enable_timing=True); e1.record()
            exposed.append((e0, e1))
        t_host.append(time.perf_counter())  # step() returned
        if host_times is not None:
            host_times.append([round((b - a) * 1e3, 1) for a, b in zip(t_host, t_host[1:])])
    return last


def timed(fn, device, wait_writeback=None):
    """Returns (event ms, host wall ms until ``fn`` returned, drain ms, fn's result).
    Bracketed by barrier + synchronize on both sides.  The closing event is recorded on
    the launching stream once every stream of the process is idle, so the event time
    includes the drain: what was still running on other streams when the launching stream
    was done (the write-back of the last step's optimizer state, which in a longer run
    overlaps the next forward pass).  ``drain`` reports that part on its own."""
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    t0 = time.perf_counter()
    e0.record()
    out = fn()
    e1.record()
    wall = time.perf_counter() - t0
    if wait_writeback is not None:
        wait_writeback()  # also waits for write-backs a helper thread has not issued yet
    torch.cuda.synchronize()
    e2.record()
    e2.synchronize()
    dist.barrier()
    return e0.elapsed_time(e2), wall * 1e3, e1.elapsed_time(e2), out


def main():
    args = parse_args()
    preset = dict(PRESETS[args.preset])
    for k in ("seq", "ga", "mode", "mb"):
        if getattr(args, k) is not None:
            preset[k] = getattr(args, k)
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "offload_adam")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return 0
    rank, local_rank, world = setup_dist(args.gpus)
    device = torch.device("cuda", local_rank)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True

    short = host_memory_shortfall(args, preset, world)
    if short is not None:
        # pinning more host memory than the machine has takes the whole node down: refuse
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": short,
                              "config": {"model": args.model, "grad_layout": args.grad_layout, "n_gpus": world}}))
        dist.barrier()
        dist.destroy_process_group()
        return 0
    build = build_ours if args.impl == "ours" else build_reference
    t_build = time.perf_counter()
    model, opt, loss_fn, vocab = build(args, preset, device)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build

    ga, seq, mb = preset["ga"], preset["seq"], preset["mb"]
    gen = torch.Generator().manual_seed(1000 + rank)
    host_batches = [torch.randint(0, vocab, (mb, seq), generator=gen, dtype=torch.long).pin_memory()
                    for _ in range(ga * 2)]
    dev_batches = [b.to(device) for b in host_batches]
    tokens_per_step = mb * seq * ga * world

    launches0 = None
    if args.impl == "ours":
        from offload_adam_b200 import _ext
        C = _ext.load(required=True)

    # warm-up (also compiles/loads every kernel)
    run_steps(args.warmup, ga, opt, loss_fn, batches_dev=dev_batches)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()

    sampler = ClockSampler(local_rank)
    sampler.start()
    moved0 = None
    if args.impl == "ours":
        launches0 = C.launch_count()
        moved0 = opt._engine.bytes_moved() if hasattr(opt, "_engine") else None
    exposed = []
    ms, wall_ms, drain_ms, _ = timed(lambda: run_steps(args.steps, ga, opt, loss_fn, batches_dev=dev_batches,
                                                       exposed=exposed), device,
                                     getattr(opt, "wait_writeback", None))
    launches = (C.launch_count() - launches0) if launches0 is not None else None
    clocks = sampler.stop()
    link_bytes = None
    moved1 = opt._engine.bytes_moved() if args.impl == "ours" and hasattr(opt, "_engine") else None
    if moved0 is not None and moved1 is not None:
        link_bytes = {"h2d": (moved1[0] - moved0[0]) / args.steps, "d2h": (moved1[1] - moved0[1]) / args.steps}
    exposed_ms = statistics.mean(a.elapsed_time(b) for a, b in exposed) if exposed else None
    ms = max_over_ranks(ms, device)
    drain_ms_all = max_over_ranks(drain_ms, device)
    exposed_ms = max_over_ranks(exposed_ms, device)
    peak_gb = torch.cuda.max_memory_allocated() / 1024**3

    if args.verbose > 2 and args.impl == "ours" and rank == 0:
        print("[rank 0] last timed step, ms from its start:", opt.trace_report(),
              "host:", getattr(opt, "host_trace", None), flush=True)
    if args.profile_range:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        run_steps(1, ga, opt, loss_fn, batches_dev=dev_batches)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()

    e2e = None
    if not args.skip_e2e:
        if args.impl == "ours":
            # the package's scalar read: a kernel store into mapped host memory, which
            # does not queue behind the optimizer's bulk write-backs in the copy engine
            from offload_adam_b200.utils.scalar import read_scalar as read_loss
        else:
            read_loss = lambda t: t.float().item()  # noqa: E731
        host_times = [] if args.verbose > 2 else None
        ms2, wall2, drain2, last_loss = timed(lambda: run_steps(args.steps, ga, opt, loss_fn, host_times=host_times,
                                                        batches_host=host_batches, device=device,
                                                        read_loss=read_loss), device,
                                              getattr(opt, "wait_writeback", None))
        ms2 = max_over_ranks(max(ms2, 0.0), device)
        wall2 = max_over_ranks(wall2, device)
        # the event time ends when the last step's kernels have run on the launching
        # stream, the wall time when the host has enqueued it; report the larger
        t = max(ms2, wall2)
        if host_times and rank == 0:
            print("[rank 0] e2e host ms per step [stage inputs + enqueue fwd/bwd, read loss, step()]:",
                  host_times, flush=True)
        e2e = {"value": tokens_per_step * args.steps / (t / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": ga * mb * seq * 8, "d2h_bytes_per_step": 4,
               "ms_per_step": t / args.steps, "loss": last_loss,
               "drain_ms_after_region": max_over_ranks(drain2, device)}

    if rank == 0:
        value = tokens_per_step * args.steps / (ms / 1e3)
        out = {
            "metric": "tokens/s (max over ranks) 8B-shape offload Adam",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform token ids; random-init weights N(0,0.02)",
            "impl": args.impl,
            "config": {
                "model": args.model + (f"-{args.layers}layers" if args.layers else ""),
                "global_batch": mb * ga * world, "seq_len": seq,
                "parallelism": f"zero1-dp{world}" if preset["optimizer"] == "distributed" else "single",
                "optimizer": ("DistributedOffloadAdam" if preset["optimizer"] == "distributed" else "OffloadAdam"),
                "mode": preset["mode"], "max_grad_norm": preset["max_grad_norm"],
                "grad_accum": ga, "micro_batch": mb, "activation_checkpointing": bool(args.grad_ckpt),
                "l2_policy": "inputs larger than L2 (16 GB of parameters per step)",
                "transfer": getattr(opt, "transfer", None),
                "grad_residency": getattr(opt, "grad_residency", "host (reference)"),
                "comm": getattr(opt, "comm", None),
                "grad_layout": getattr(opt, "grad_layout", None),
                "quant": args.quant,
                "staging_gib": (getattr(getattr(opt, "_engine", None), "staging_bytes", 0) or 0) / 2**30,
                "resident_gib": (getattr(getattr(opt, "_engine", None), "resident_bytes", 0) or 0) / 2**30,
                "resident_writeback": getattr(opt, "resident_writeback", None),
                "model_impl": (args.model_impl + ("+chunked_loss" if args.hf_chunked_loss and args.model_impl == "hf" else ""))
                if args.impl == "ours" else "hf",
            },
            "optimizer_link_bytes_per_step": link_bytes,
            "exposed_opt_ms": exposed_ms, "peak_gpu_gb": peak_gb, "build_s": t_build,
            "optimizer_memory_bytes": opt.memory_report() if hasattr(opt, "memory_report") else None,
            "wall_ms_per_step": wall_ms / args.steps,
            "drain_ms_after_region": drain_ms_all,
            "timing": "CUDA events on the launching stream, barrier + synchronize on both sides; the closing "
                      "event is recorded after all streams drained, so the write-back of the last step's "
                      "optimizer state (drain_ms_after_region, part of the timed region) is included",
            "clocks": clocks,
            "e2e": e2e, "gpu_launches": launches,
        }
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
