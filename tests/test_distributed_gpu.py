"""ZeRO-1 on real GPUs (needs at least two): the symmetric-memory path (peer pull +
fused Adam + push, no NCCL on the hot path) against a single-GPU restatement of the
same schedule, bit for bit, and against the torch.distributed path.  Ranks run as
child processes; NVLS is off and device-side waits are bounded."""

import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

pytestmark = pytest.mark.gpu


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(256, 512, bias=True)
        self.n = nn.LayerNorm(512)
        self.b = nn.Linear(512, 256, bias=False)
        self.c = nn.Linear(256, 15, bias=False)  # 15 rows: replicated, takes the collective path

    def forward(self, x):
        return self.c(torch.relu(self.b(self.n(torch.relu(self.a(x))))))


def make_net(device):
    torch.manual_seed(0)
    return Net().to(torch.bfloat16).to(device)


def rank_batches(rank, n, device):
    g = torch.Generator().manual_seed(100 + rank)
    return [torch.randn(16, 256, generator=g).to(torch.bfloat16).to(device) for _ in range(n)]


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def bf16_accumulate(model, batches, ga):
    acc = None
    for b in batches:
        model.zero_grad()
        (model(b).float().pow(2).mean() / ga).backward()
        gs = [p.grad.detach().clone() for p in model.parameters()]
        acc = gs if acc is None else [(a.float() + g.float()).to(torch.bfloat16) for a, g in zip(acc, gs)]
    return acc


def restatement(device, world, mode, clip, ga, steps):
    """Every rank's work replayed on one GPU + rank-ordered fp32 averaging."""
    from offload_adam_b200 import Adam
    from offload_adam_b200.ops.adam_step import adam_step
    model = make_net(device)
    ref = Adam(model.parameters(), lr=1e-2, weight_decay=0.05, mode=mode, decoupled_weight_decay=True)
    data = [rank_batches(r, ga * steps, device) for r in range(world)]
    scale = torch.tensor(1.0 / world, dtype=torch.float32, device=device)
    for s in range(steps):
        per_rank = [bf16_accumulate(model, data[r][s * ga:(s + 1) * ga], ga) for r in range(world)]
        avg = []
        for parts in zip(*per_rank):
            f = torch.zeros_like(parts[0], dtype=torch.float32)
            for g in parts:
                f = f + g.float()
            avg.append((f * scale).to(torch.bfloat16))
        coef = None
        if clip is not None:
            total = torch.sqrt(sum((g.float() ** 2).sum() for g in avg))
            coef = torch.clamp(clip / (total + 1e-6), max=1.0).reshape(1)
        for p, g in zip(model.parameters(), avg):
            st = ref.state[p]
            ref._init_state_if_empty(p, st)
            st["step"] += 1
            tensors = {k: st[k] for k in ref.config["states"]}
            tensors["grad"] = g
            adam_step(mode, p.data, tensors, 1e-2, 0.05, 0.9, 0.999, 1e-8, st["step"],
                      decoupled_weight_decay=True, clip_coef=coef)
    return [p.detach().clone() for p in model.parameters()]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    report = {}
    try:
        from offload_adam_b200 import DistributedOffloadAdam
        ga, steps = 2, 3
        for mode in ("fp32_master", "fp31_master"):
            for clip in (None, 0.05):
                results = {}
                for comm in ("symm", "nccl"):
                    model = make_net(device)
                    opt = DistributedOffloadAdam(model, lr=1e-2, weight_decay=0.05, mode=mode, max_grad_norm=clip,
                                                 decoupled_weight_decay=True, inplace_param_threshold=2000,
                                                 comm=comm, wait_timeout_ms=20000, chunk_elems=4096, ring_slots=3)
                    assert opt.comm == comm
                    data = rank_batches(rank, ga * steps, device)
                    k = 0
                    for _ in range(steps):
                        for micro in range(ga):
                            opt.ready_for_optimizer_step = micro == ga - 1
                            (model(data[k]).float().pow(2).mean() / ga).backward()
                            k += 1
                        opt.step()
                    opt.synchronize()
                    results[comm] = [p.detach().clone() for p in model.parameters()]
                    # replicas must be identical on all ranks
                    for p in results[comm]:
                        gathered = [torch.empty_like(p) for _ in range(world)]
                        dist.all_gather(gathered, p.contiguous())
                        assert all(torch.equal(gathered[0], g) for g in gathered), (mode, clip, comm, "replicas differ")
                want = restatement(device, world, mode, clip, ga, steps)
                exact = all(torch.equal(a, b) for a, b in zip(results["symm"], want))
                # NCCL averages bf16 in its own order and precision: after a few Adam steps
                # single elements may differ by whole updates (lr = 1e-2), the bulk agrees
                close = all((a.float() - b.float()).abs().mean().item() < 2e-3 and
                            (a.float() - b.float()).abs().max().item() < 0.1
                            for a, b in zip(results["symm"], results["nccl"]))
                near = all(torch.allclose(a.float(), b.float(), atol=4e-3, rtol=0)
                           for a, b in zip(results["symm"], want))
                report[f"{mode}/{clip}"] = {"exact": exact, "close_to_nccl": close, "near": near}
    finally:
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.destroy_process_group()


def test_symm_path_matches_restatement_and_collectives():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, free_port(), d), nprocs=world, join=True)
        reports = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(world)]
    for rep in reports:
        assert len(rep) == 4
        for key, r in rep.items():
            assert r["close_to_nccl"] and r["near"], (key, r)
            if key.endswith("/None"):
                # without clipping there is no cross-rank scalar: bit-exact by construction
                assert r["exact"], (key, r)


# ------------------------------------------- sharded QAT: owners quantize, packed rows travel
class QNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(256, 512, bias=False)
        self.l2 = nn.Linear(512, 256, bias=False)

    def forward(self, x):
        return self.l2(torch.relu(self.l1(x)))


def _bits(t):
    return t.view(torch.uint8) if t.element_size() == 1 else t


def _qat_worker(rank, world, port, out_dir):  # noqa: C901
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    report = {}
    try:
        from offload_adam_b200 import DistributedOffloadAdam
        from offload_adam_b200.qweight import (Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight,
                                               quantize_linears)
        for name, cls in (("nvfp4", NVFP4QWeight), ("nf4", NF4QWeight), ("int4", Int4QWeight),
                          ("int8", Int8QWeight)):
            for comm, clip in (("nccl", 1.0), ("symm", 1.0), ("symm", None)):
                torch.manual_seed(0)
                model = QNet().to(torch.bfloat16).to(device)
                quantize_linears(model, cls)
                # small chunks: every shard streams through the staging buffer in several pieces
                opt = DistributedOffloadAdam(model, lr=1e-2, weight_decay=0.01, mode="fp32_master",
                                             max_grad_norm=clip, decoupled_weight_decay=True, comm=comm,
                                             chunk_elems=16384, wait_timeout_ms=20000,
                                             keep_resident=(clip is None))
                assert opt.comm == comm
                if comm == "symm":
                    assert all(opt._symm.handles(p) and opt._fused_quant_plan(p) is not None
                               for p in model.parameters())
                g = torch.Generator().manual_seed(7 + rank)
                for _ in range(3):
                    for micro in range(2):
                        opt.ready_for_optimizer_step = micro == 1
                        x = torch.randn(8, 256, generator=g).to(torch.bfloat16).to(device)
                        (model(x).float().pow(2).mean() / 2).backward()
                    opt.step()
                opt.synchronize()
                ok = True
                for p in model.parameters():
                    shard = opt.state[p]["master_params"].to(device)
                    full = torch.empty(p.shape, dtype=torch.float32, device=device)
                    dist.all_gather_into_tensor(full.view(-1), shard.view(-1))
                    want = cls.from_float(torch.zeros(p.shape, dtype=torch.bfloat16, device=device))
                    want.copy_(full)  # the gather-fp32-and-requantize-everything route
                    ok = ok and all(torch.equal(_bits(a), _bits(b))
                                    for a, b in zip(p.data._payload(), want._payload()))
                    # every replica holds the same packed weight
                    for t in p.data._payload():
                        mine = _bits(t).contiguous()
                        both = [torch.empty_like(mine) for _ in range(world)]
                        dist.all_gather(both, mine)
                        ok = ok and all(torch.equal(both[0], b) for b in both)
                report[f"{name}/{comm}/{clip}"] = ok
                del opt, model
                torch.cuda.synchronize()
                dist.barrier()
    finally:
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.destroy_process_group()


def test_sharded_qat_payload_matches_full_requantization():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_qat_worker, args=(2, free_port(), d), nprocs=2, join=True)
        reports = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(2)]
    for rep in reports:
        assert len(rep) == 12 and all(rep.values()), rep


# ------------------------------------ shard-sized gradient accumulators on the peer path
def restatement_shard_layout(device, world, clip, ga, steps):
    """grad_layout='shard' replayed on one GPU: every micro-batch's gradient is averaged
    over the ranks first (fp32 sum in rank order, one rounding), then added to the
    accumulator in bf16."""
    from offload_adam_b200 import Adam
    from offload_adam_b200.ops.adam_step import adam_step
    mode = "fp32_master"
    model = make_net(device)
    ref = Adam(model.parameters(), lr=1e-2, weight_decay=0.05, mode=mode, decoupled_weight_decay=True)
    data = [rank_batches(r, ga * steps, device) for r in range(world)]
    scale = torch.tensor(1.0 / world, dtype=torch.float32, device=device)
    params = list(model.parameters())
    sharded = [p.dim() >= 1 and p.shape[0] % world == 0 and p.numel() >= 2000 for p in params]
    for s in range(steps):
        acc = [None] * len(params)
        full = [[None] * len(params) for _ in range(world)]  # tensors that keep full-shape accumulators
        for micro in range(ga):
            per_rank = []
            for r in range(world):
                model.zero_grad()
                (model(data[r][s * ga + micro]).float().pow(2).mean() / ga).backward()
                per_rank.append([p.grad.detach().clone() for p in params])
            for i in range(len(params)):
                if sharded[i]:
                    f = torch.zeros_like(per_rank[0][i], dtype=torch.float32)
                    for r in range(world):
                        f = f + per_rank[r][i].float()
                    mean = (f * scale).to(torch.bfloat16)
                    acc[i] = mean if acc[i] is None else (acc[i].float() + mean.float()).to(torch.bfloat16)
                else:
                    for r in range(world):
                        g = per_rank[r][i]
                        full[r][i] = g if full[r][i] is None else (full[r][i].float() + g.float()).to(torch.bfloat16)
        for i in range(len(params)):
            if not sharded[i]:
                f = torch.zeros_like(full[0][i], dtype=torch.float32)
                for r in range(world):
                    f = f + full[r][i].float()
                acc[i] = (f * scale).to(torch.bfloat16)
        coef = None
        if clip is not None:
            total = torch.sqrt(sum((g.float() ** 2).sum() for g in acc))
            coef = torch.clamp(clip / (total + 1e-6), max=1.0).reshape(1)
        for p, g in zip(params, acc):
            st = ref.state[p]
            ref._init_state_if_empty(p, st)
            st["step"] += 1
            tensors = {k: st[k] for k in ref.config["states"]}
            tensors["grad"] = g
            adam_step(mode, p.data, tensors, 1e-2, 0.05, 0.9, 0.999, 1e-8, st["step"],
                      decoupled_weight_decay=True, clip_coef=coef)
    return [p.detach().clone() for p in params]


def _shard_layout_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    report = {}
    try:
        from offload_adam_b200 import DistributedOffloadAdam
        ga, steps = 3, 3
        for clip in (None, 0.05):
            model = make_net(device)
            opt = DistributedOffloadAdam(model, lr=1e-2, weight_decay=0.05, mode="fp32_master", max_grad_norm=clip,
                                         decoupled_weight_decay=True, inplace_param_threshold=2000, comm="symm",
                                         grad_layout="shard", wait_timeout_ms=20000, chunk_elems=4096)
            assert opt.comm == "symm" and opt._symm.shard_layout
            data = rank_batches(rank, ga * steps, device)
            k = 0
            for _ in range(steps):
                for micro in range(ga):
                    opt.ready_for_optimizer_step = micro == ga - 1
                    (model(data[k]).float().pow(2).mean() / ga).backward()
                    k += 1
                opt.step()
            opt.synchronize()
            got = [p.detach().clone() for p in model.parameters()]
            want = restatement_shard_layout(device, world, clip, ga, steps)
            same_everywhere = True
            for p in got:
                gathered = [torch.empty_like(p) for _ in range(world)]
                dist.all_gather(gathered, p.contiguous())
                same_everywhere = same_everywhere and all(torch.equal(gathered[0], g) for g in gathered)
            report[str(clip)] = {
                "replicas_equal": same_everywhere,
                "exact": all(torch.equal(a, b) for a, b in zip(got, want)),
                "near": all(torch.allclose(a.float(), b.float(), atol=4e-3, rtol=0) for a, b in zip(got, want)),
            }
            del opt, model
            torch.cuda.synchronize()
            dist.barrier()
    finally:
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.destroy_process_group()


def test_shard_gradient_layout_on_the_peer_path_matches_its_restatement():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_shard_layout_worker, args=(world, free_port(), d), nprocs=world, join=True)
        reports = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(world)]
    for rep in reports:
        assert set(rep) == {"None", "0.05"}, rep
        for key, r in rep.items():
            assert r["replicas_equal"] and r["near"], (key, r)
            if key == "None":
                assert r["exact"], (key, r)


# --------------------------------- a parameter that gets no gradient must not stall the step
class Branchy(nn.Module):
    def __init__(self):
        super().__init__()
        self.used = nn.Linear(256, 256, bias=False)
        self.unused = nn.Linear(256, 256, bias=False)

    def forward(self, x):
        return self.used(x)


def _unused_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    report = {"ok": False}
    try:
        from offload_adam_b200 import DistributedOffloadAdam
        for clip in (None, 1.0):
            torch.manual_seed(0)
            model = Branchy().to(torch.bfloat16).to(device)
            before = model.unused.weight.detach().clone()
            opt = DistributedOffloadAdam(model, lr=1e-2, mode="fp32_master", max_grad_norm=clip, comm="symm",
                                         inplace_param_threshold=0, wait_timeout_ms=3000)
            x = torch.randn(8, 256, device=device).to(torch.bfloat16)
            for _ in range(2):
                opt.ready_for_optimizer_step = True
                model(x).float().pow(2).mean().backward()
                opt.step()
            opt.synchronize()  # raises if a bounded wait gave up
            assert torch.equal(model.unused.weight, before)
            assert opt.state[model.unused.weight]["step"] == 0 and opt.state[model.used.weight]["step"] == 2
            del opt, model
            dist.barrier()
        report["ok"] = True
    finally:
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.destroy_process_group()


def test_parameter_without_gradient_does_not_stall_the_peer_path():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_unused_worker, args=(2, free_port(), d), nprocs=2, join=True)
        reports = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(2)]
    assert all(r["ok"] for r in reports), reports


# ----------------------- a model created directly in symmetric memory is adopted, not copied
def _adopt_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    report = {"ok": False}
    try:
        from offload_adam_b200 import DistributedOffloadAdam
        from offload_adam_b200.models.llama import build_llama, tiny_llama
        cfg = tiny_llama()
        plain = build_llama(cfg, device=device, seed=0)
        symm = build_llama(cfg, device=device, seed=0, symmetric_group=dist.group.WORLD, symmetric_threshold=1000)
        symm.load_state_dict(plain.state_dict())
        kw = dict(lr=1e-3, mode="fp32_master", max_grad_norm=1.0, comm="symm", grad_layout="shard",
                  inplace_param_threshold=1000, wait_timeout_ms=20000, chunk_elems=16384)
        o_plain = DistributedOffloadAdam(plain, **kw)
        o_symm = DistributedOffloadAdam(symm, **kw)
        assert o_symm._symm.adopted_param_arena and not o_plain._symm.adopted_param_arena
        g = torch.Generator().manual_seed(50 + rank)
        for _ in range(2):
            for micro in range(2):
                ids = torch.randint(0, cfg.vocab_size, (2, 64), generator=g).to(device)
                for model, opt in ((plain, o_plain), (symm, o_symm)):
                    opt.ready_for_optimizer_step = micro == 1
                    (model(ids, labels=ids) / 2).backward()
            o_plain.step()
            o_symm.step()
        o_plain.synchronize()
        o_symm.synchronize()
        assert all(torch.equal(a, b) for a, b in zip(plain.parameters(), symm.parameters()))
        report["ok"] = True
    finally:
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.destroy_process_group()


def test_model_built_in_symmetric_memory_is_adopted():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_adopt_worker, args=(2, free_port(), d), nprocs=2, join=True)
        reports = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(2)]
    assert all(r["ok"] for r in reports), reports


# ------------- torch.distributed back end with gradients on the host (both gradient layouts)
def _host_grad_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    report = {}
    try:
        from offload_adam_b200 import DistributedOffloadAdam
        ga, steps = 3, 3
        for layout in ("full", "shard"):
            for clip in (None, 0.05):
                results = {}
                for residency in ("host", "device"):
                    model = make_net(device)
                    opt = DistributedOffloadAdam(model, lr=1e-2, weight_decay=0.05, mode="fp32_master",
                                                 max_grad_norm=clip, decoupled_weight_decay=True,
                                                 inplace_param_threshold=2000, comm="nccl", grad_layout=layout,
                                                 grad_residency=residency, chunk_elems=4096, ring_slots=3)
                    assert opt.comm == "nccl" and opt.grad_residency == residency
                    data = rank_batches(rank, ga * steps, device)
                    k = 0
                    for _ in range(steps):
                        for micro in range(ga):
                            opt.ready_for_optimizer_step = micro == ga - 1
                            (model(data[k]).float().pow(2).mean() / ga).backward()
                            k += 1
                        opt.step()
                    opt.synchronize()
                    results[residency] = [p.detach().clone() for p in model.parameters()]
                # the kernels that read the pinned gradient buffer wait for the copy that filled it:
                # gradients parked on the host must give the bits of gradients kept in HBM
                report[f"{layout}/{clip}"] = all(torch.equal(a, b)
                                                 for a, b in zip(results["host"], results["device"]))
    finally:
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.destroy_process_group()


def test_host_resident_gradients_on_the_collective_path_match_device_resident_ones():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_host_grad_worker, args=(2, free_port(), d), nprocs=2, join=True)
        reports = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(2)]
    for rep in reports:
        assert len(rep) == 4 and all(rep.values()), rep
