"""Gradient kernels (accumulate + squared norm, clip coefficient) and the pinned arena."""

import pytest
import torch

from offload_adam_b200 import _ext
from offload_adam_b200.ops import grad_ops
from offload_adam_b200.utils import pinned_alloc


# ------------------------------------------------------------------------- CPU
def test_cpu_accumulate_and_clip():
    a = (torch.randn(1000) * 0.1).to(torch.bfloat16)
    b = (torch.randn(1000) * 0.1).to(torch.bfloat16)
    out = torch.empty_like(a)
    sq = torch.zeros(1)
    grad_ops.grad_accumulate(out, a, b, sumsq=sq)
    want = (a.float() + b.float()).to(torch.bfloat16)
    assert torch.equal(out, want)
    assert torch.allclose(sq, (want.float() ** 2).sum().reshape(1))
    slots = torch.tensor([4.0, 5.0, 16.0])
    cn = torch.zeros(2)
    grad_ops.clip_finalize(slots, None, None, 1.0, coef_norm=cn)
    assert torch.allclose(cn, torch.tensor([1.0 / (5.0 + 1e-6), 5.0]))
    grad_ops.clip_finalize(slots, torch.tensor([0, 1], dtype=torch.int32), torch.tensor([7.0]), 100.0, coef_norm=cn)
    assert torch.allclose(cn, torch.tensor([1.0, 4.0]))


def test_arena_without_cuda_registration():
    specs = [((3, 5), torch.bfloat16), ((1000,), torch.float32), ((7,), torch.int16), ((0,), torch.float32)]
    arena = pinned_alloc.PinnedArena(specs, numa_node=None, register_cuda=False, segment_bytes=8192)
    ts = list(arena.tensors())
    assert [tuple(t.shape) for t in ts] == [(3, 5), (1000,), (7,), (0,)]
    assert [t.dtype for t in ts] == [torch.bfloat16, torch.float32, torch.int16, torch.float32]
    for t in ts:
        assert t.data_ptr() % 256 == 0
        assert float(t.float().abs().sum()) == 0.0
    ts[1].fill_(3.0)
    assert ts[1].sum().item() == 3000.0 and ts[0].float().sum().item() == 0.0
    st = arena.stats()
    assert st["segments"] >= 1 and st["registered"] is False and st["numa_bound"] is False
    # tensors keep the mapping alive after the arena object is gone
    del arena
    ts[1].add_(1.0)
    assert ts[1][0].item() == 4.0


def test_arena_binds_to_a_numa_node_with_raw_syscall():
    C = _ext.load(required=False)
    if C is None or C.numa_num_nodes() < 1:
        pytest.skip("no NUMA information")
    arena = pinned_alloc.PinnedArena([((1 << 16,), torch.float32)], numa_node=0, register_cuda=False)
    assert arena.stats()["numa_bound"] is True and arena.stats()["numa_node"] == 0
    assert pinned_alloc.numa_node_free_bytes(0) > 0
    assert pinned_alloc.numa_node_free_bytes(4095) is None


@pytest.mark.parametrize("call", ["mmap", "mbind"])
def test_arena_failure_injection_releases_and_raises(call):
    C = _ext.load(required=False)
    if C is None:
        pytest.skip("extension not built")
    try:
        # second segment fails: the first one must be released, nothing leaks or faults
        C.arena_inject_failure(call, 1)
        with pytest.raises(RuntimeError, match=call):
            pinned_alloc.PinnedArena([((4096,), torch.float32)] * 4, numa_node=0 if call == "mbind" else None,
                                     register_cuda=False, segment_bytes=16384)
    finally:
        C.arena_reset_syscalls()
    ok = pinned_alloc.PinnedArena([((16,), torch.float32)], numa_node=None, register_cuda=False)
    assert ok.tensor(0).numel() == 16


def test_resolve_numa_target():
    assert pinned_alloc.resolve_numa_target(None) is None
    assert pinned_alloc.resolve_numa_target(3) == 3
    with pytest.raises(ValueError):
        pinned_alloc.resolve_numa_target("nope")
    if not torch.cuda.is_available():
        assert pinned_alloc.resolve_numa_target("auto") is None
        assert pinned_alloc.gpu_numa_node() == -1


# ------------------------------------------------------------------------- GPU
@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 9, 4096, 100003, 1 << 22])
def test_gpu_accumulate_sumsq_bitwise_and_deterministic(n):
    a = (torch.randn(n) * 0.1).to(torch.bfloat16).cuda()
    b = (torch.randn(n) * 0.1).to(torch.bfloat16).cuda()
    out = torch.empty_like(a)
    sq = torch.zeros(1, device="cuda")
    scratch = grad_ops.sumsq_scratch("cuda")
    grad_ops.grad_accumulate(out, a, b, sumsq=sq, scratch=scratch)
    want = (a.float() + b.float()).to(torch.bfloat16)
    assert torch.equal(out, want)
    ref = (want.double() ** 2).sum().item()
    assert abs(sq.item() - ref) <= 2e-6 * max(ref, 1e-30) + 1e-12
    first = sq.clone()
    for _ in range(3):
        grad_ops.grad_accumulate(None, want, None, sumsq=sq, scratch=scratch)
        assert torch.equal(sq, first)  # fixed reduction order
    grad_ops.grad_accumulate(None, want, None, sumsq=sq, sumsq_accumulate=True, scratch=scratch)
    assert abs(sq.item() - 2 * first.item()) <= 1e-6 * first.item()


@pytest.mark.gpu
def test_gpu_clip_finalize():
    slots = torch.tensor([4.0, 5.0, 16.0], device="cuda")
    cn = torch.zeros(2, device="cuda")
    grad_ops.clip_finalize(slots, None, None, 1.0, coef_norm=cn)
    assert torch.allclose(cn.cpu(), torch.tensor([1.0 / (5.0 + 1e-6), 5.0]))
    tot = torch.zeros(1, device="cuda")
    grad_ops.clip_finalize(slots, torch.tensor([0, 2], dtype=torch.int32, device="cuda"), None, 1.0, total_sq=tot)
    assert tot.item() == 20.0
    grad_ops.clip_finalize(None, None, tot, 100.0, coef_norm=cn)
    assert cn[0].item() == 1.0


@pytest.mark.gpu
def test_arena_is_pinned_and_device_mapped():
    arena = pinned_alloc.PinnedArena([((1 << 20,), torch.bfloat16), ((1 << 20,), torch.float32)], numa_node="auto")
    g, m = arena.tensors()
    assert g.is_pinned() and m.is_pinned() and arena.stats()["registered"]
    src = torch.randn(1 << 20, device="cuda").to(torch.bfloat16)
    # zero-copy kernel writes straight into the host buffer
    grad_ops.grad_accumulate(g, src, None)
    torch.cuda.synchronize()
    assert torch.equal(g, src.cpu())
    sq = torch.zeros(1, device="cuda")
    grad_ops.grad_accumulate(g, src, g, sumsq=sq, scratch=grad_ops.sumsq_scratch("cuda"))
    torch.cuda.synchronize()
    assert torch.equal(g, (src.float() * 2).to(torch.bfloat16).cpu())
    t = pinned_alloc.zeros_pinned((5, 7), torch.int16)
    assert t.is_pinned() and t.shape == (5, 7) and int(t.abs().sum()) == 0


@pytest.mark.gpu
def test_read_scalar_bypasses_copy_engine():
    from offload_adam_b200.utils.scalar import read_scalar
    assert read_scalar(torch.tensor(3.25, device="cuda")) == 3.25
    assert read_scalar(torch.tensor([-7.5], device="cuda", dtype=torch.bfloat16)) == -7.5
    assert read_scalar(torch.tensor(1.5)) == 1.5
