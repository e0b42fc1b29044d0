"""Peer-memory kernels of the ZeRO-1 path, exercised on ONE GPU: the "replicas of the
other ranks" are ordinary buffers of the same device, which is all the kernels need
(they only see addresses).  Bounded waits are driven to their limit with a flag that
nothing sets and must come back with a status code, never hang."""

import time

import pytest
import torch

from offload_adam_b200 import _ext
from offload_adam_b200.ops import grad_ops
from offload_adam_b200.ops.adam_step import adam_step

pytestmark = pytest.mark.gpu

MODES = ["stochastic_rounding", "fp32_master", "fp31_master", "fp32_master_custom_rounding"]


def ref_average(grads):
    acc = torch.zeros_like(grads[0], dtype=torch.float32)
    for g in grads:  # rank order, fp32
        acc = acc + g.float()
    scale = torch.tensor(1.0 / len(grads), dtype=torch.float32, device=acc.device)
    return (acc * scale).to(torch.bfloat16)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("n", [5, 4096, 100003])
def test_peer_reduce_matches_rank_ordered_fp32_average(world, n):
    C = _ext.load(required=True)
    torch.manual_seed(world * 1000 + n)
    grads = [(torch.randn(n, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(world)]
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    sq = torch.zeros(1, device="cuda")
    scratch = grad_ops.sumsq_scratch("cuda")
    C.peer_reduce(out, [g.data_ptr() for g in grads], 1.0 / world, sq, scratch)
    want = ref_average(grads)
    assert torch.equal(out, want)
    ref_sq = (want.double() ** 2).sum().item()
    assert abs(sq.item() - ref_sq) <= 2e-6 * ref_sq + 1e-12
    again = torch.zeros(1, device="cuda")
    C.peer_reduce(out, [g.data_ptr() for g in grads], 1.0 / world, again, scratch)
    assert torch.equal(sq, again)  # fixed reduction order


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("world", [2, 8])
def test_fused_pull_adam_push_equals_separate_steps(mode, world):
    """One launch (pull + average + Adam + push) == reduce, then Adam, then copies."""
    n = 16 * 1000 + 7
    torch.manual_seed(world)
    grads = [(torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16) for _ in range(world)]

    def fresh():
        g = torch.Generator(device="cuda").manual_seed(5)
        p = (torch.randn(n, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        st = {"exp_avg": (torch.randn(n, device="cuda", generator=g) * 1e-3).to(torch.bfloat16),
              "exp_avg_sq": (torch.rand(n, device="cuda", generator=g) * 1e-5).to(torch.bfloat16)}
        if mode == "fp32_master":
            st["master_params"] = p.float() + 1e-5
        elif mode != "stochastic_rounding":
            st["rounding_error"] = torch.randint(-3000, 3000, (n,), device="cuda", generator=g).to(torch.int16)
        return p, st

    hp = (1e-3, 0.01, 0.9, 0.999, 1e-8, 3)
    clip = torch.tensor([0.7], device="cuda")
    p1, st1 = fresh()
    st1["grad"] = ref_average(grads)
    adam_step(mode, p1, st1, *hp, decoupled_weight_decay=True, seed=9, clip_coef=clip)

    p2, st2 = fresh()
    replicas = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    adam_step(mode, p2, st2, *hp, decoupled_weight_decay=True, seed=9, clip_coef=clip, use_cuda=True,
              g_peers=[g.data_ptr() for g in grads], g_scale=1.0 / world,
              p_peers=[r.data_ptr() for r in replicas])
    torch.cuda.synchronize()
    for r in replicas:
        assert torch.equal(r, p1)
    for k in st2:
        assert torch.equal(st2[k], st1[k]), k
    # push only (the clip path): local, already reduced gradient + stores into all replicas
    p3, st3 = fresh()
    st3["grad"] = ref_average(grads)
    replicas = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    adam_step(mode, p3, st3, *hp, decoupled_weight_decay=True, seed=9, clip_coef=clip,
              p_peers=[r.data_ptr() for r in replicas])
    torch.cuda.synchronize()
    for r in replicas:
        assert torch.equal(r, p1)
    assert torch.equal(st3["exp_avg"], st1["exp_avg"])


def test_staged_engine_with_peers_matches_direct():
    from offload_adam_b200.engine import TransferEngine
    from offload_adam_b200.utils.pinned_alloc import PinnedArena
    n, world = 5000, 4
    grads = [(torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16) for _ in range(world)]
    arena = PinnedArena([((n,), torch.bfloat16), ((n,), torch.bfloat16), ((n,), torch.float32)], numa_node=None)
    m, v, master = arena.tensors()
    master.copy_(torch.randn(n) * 0.05)
    ref_states = {"grad": ref_average(grads), "exp_avg": m.cuda(), "exp_avg_sq": v.cuda(), "master_params": master.cuda()}
    p_ref = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    adam_step("fp32_master", p_ref, ref_states, 1e-3, 0.0, 0.9, 0.999, 1e-8, 1)
    eng = TransferEngine("cuda", "fp32_master", 1, transfer="staged", chunk_elems=1024, ring_slots=3)
    replicas = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    eng.step(0, None, None, None, {"exp_avg": m, "exp_avg_sq": v, "master_params": master},
             (1e-3, 0.0, 0.9, 0.999, 1e-8), 1, False,
             g_peers=[g.data_ptr() for g in grads], g_scale=1.0 / world, p_peers=[r.data_ptr() for r in replicas])
    eng.synchronize()
    for r in replicas:
        assert torch.equal(r, p_ref)
    assert torch.equal(master, ref_states["master_params"].cpu())
    assert torch.equal(m, ref_states["exp_avg"].cpu())


def test_signal_and_wait_flags():
    C = _ext.load(required=True)
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32).pin_memory()
    base = flags.data_ptr()
    C.signal([base + 4 * i for i in (3, 4, 5)], 7)
    torch.cuda.synchronize()
    assert flags[3:6].tolist() == [7, 7, 7] and flags.sum().item() == 21
    C.wait_flags(flags, 3, 3, 7, 1000.0, status, C.SYMM_TIMEOUT_GRAD)
    C.wait_flags(flags, 3, 3, 5, 1000.0, status, C.SYMM_TIMEOUT_GRAD)  # older epoch also satisfied
    torch.cuda.synchronize()
    assert status[0].item() == 0


def test_wait_gives_up_with_status_and_later_kernels_do_nothing():
    """A flag nobody sets: the wait returns after its limit with a code, the context
    stays usable, and kernels given the status word skip their work."""
    C = _ext.load(required=True)
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32).pin_memory()
    t0 = time.perf_counter()
    C.wait_flags(flags, 0, 8, 1, 50.0, status, C.SYMM_TIMEOUT_GRAD)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert status[0].item() == C.SYMM_TIMEOUT_GRAD
    assert 0.04 <= waited < 5.0
    n = 4096
    p = torch.ones(n, dtype=torch.bfloat16, device="cuda")
    st = {"grad": torch.ones(n, dtype=torch.bfloat16, device="cuda"),
          "exp_avg": torch.zeros(n, dtype=torch.bfloat16, device="cuda"),
          "exp_avg_sq": torch.zeros(n, dtype=torch.bfloat16, device="cuda")}
    adam_step("stochastic_rounding", p, st, 1e-1, 0.0, 0.9, 0.999, 1e-8, 1, seed=1, status=status)
    out = torch.full((n,), 3.0, dtype=torch.bfloat16, device="cuda")
    C.peer_reduce(out, [p.data_ptr()], 1.0, None, None, status)
    C.wait_flags(flags, 0, 8, 1, 50.0, status, C.SYMM_TIMEOUT_PARAM)  # returns at once, keeps first code
    torch.cuda.synchronize()
    assert bool((p == 1).all()) and bool((st["exp_avg"] == 0).all()) and bool((out == 3).all())
    assert status[0].item() == C.SYMM_TIMEOUT_GRAD
    # the device is still healthy
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_scalar_exchange_single_rank_and_timeout():
    C = _ext.load(required=True)
    slots = torch.zeros(8, dtype=torch.float32, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32).pin_memory()
    mine = torch.tensor([2.5], device="cuda")
    out = torch.zeros(1, device="cuda")
    C.scalar_exchange(mine, [slots.data_ptr()], [flags.data_ptr()], slots, flags, 0, 1, 100.0, status, out)
    torch.cuda.synchronize()
    assert out.item() == 2.5 and status[0].item() == 0
    # two "ranks" on one device where the second never shows up
    C.scalar_exchange(mine, [slots.data_ptr(), slots.data_ptr()], [flags.data_ptr(), flags.data_ptr()],
                      slots, flags, 0, 2, 30.0, status, out)
    torch.cuda.synchronize()
    assert status[0].item() == C.SYMM_TIMEOUT_SCALAR
