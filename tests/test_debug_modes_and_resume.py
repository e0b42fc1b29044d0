"""Debugging aids and host-state hand-offs of the offloaded optimizer: the serialized
mode against the overlapped run, NVTX ranges, waiting for write-backs, and resuming
into an optimizer that has already loaded state for its next step ahead of time; state that
stays resident in the staging buffer against state that streams through it."""

import copy

import pytest
import torch

from offload_adam_b200 import OffloadAdam

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


class Wide(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = torch.nn.ModuleList([torch.nn.Linear(128, 128, bias=False) for _ in range(4)])

    def forward(self, x):
        for layer in self.layers:
            x = torch.relu(layer(x))
        return x


def net(device):
    torch.manual_seed(0)
    return Wide().to(torch.bfloat16).to(device)


def data(n, device):
    g = torch.Generator().manual_seed(11)
    return [torch.randn(8, 128, generator=g).to(torch.bfloat16).to(device) for _ in range(n)]


def one_step(model, opt, batches):
    for i, b in enumerate(batches):
        opt.ready_for_optimizer_step = i == len(batches) - 1
        (model(b).float().pow(2).mean() / len(batches)).backward()
    opt.step()


KW = dict(lr=1e-2, weight_decay=0.05, mode="fp32_master", decoupled_weight_decay=True,
          inplace_param_threshold=100, chunk_elems=4096)


def same(model_a, opt_a, model_b, opt_b):
    for p, q in zip(model_a.parameters(), model_b.parameters()):
        assert torch.equal(p, q)
        for k in ("exp_avg", "exp_avg_sq", "master_params"):
            assert torch.equal(opt_a.state[p][k].cpu(), opt_b.state[q][k].cpu()), k


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("clip", [None, 0.05])
def test_serialized_run_equals_overlapped_run(device, clip):
    batches = data(8, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=clip, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=clip, debug_serialize=True, nvtx=True, **KW)
    for s in range(4):
        one_step(m_a, o_a, batches[2 * s:2 * s + 2])
        one_step(m_b, o_b, batches[2 * s:2 * s + 2])
    o_a.synchronize()
    o_b.synchronize()
    same(m_a, o_a, m_b, o_b)


@pytest.mark.parametrize("device", DEVICES)
def test_wait_writeback_makes_host_state_current(device):
    batches = data(4, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=1.0, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=1.0, **KW)
    for s in range(2):
        one_step(m_a, o_a, batches[2 * s:2 * s + 2])
        one_step(m_b, o_b, batches[2 * s:2 * s + 2])
    o_a.wait_writeback()   # host state is complete; early loads of the next step may go on
    o_b.synchronize()
    if device == "cuda":
        torch.cuda.current_stream().synchronize()  # parameters are updated on the main stream's order
    same(m_a, o_a, m_b, o_b)


@pytest.mark.parametrize("device", DEVICES)
def test_resume_into_an_optimizer_that_already_loaded_ahead(device):
    """B has taken a step, so its engine has started loading state for the next one.
    Loading A's checkpoint into B must drop those copies: the next step of B has to
    match A's next step bit for bit."""
    batches = data(8, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=1.0, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=1.0, **KW)
    one_step(m_a, o_a, batches[0:2])
    one_step(m_a, o_a, batches[2:4])
    one_step(m_b, o_b, batches[4:6])  # different data: B's state differs from A's
    sd = copy.deepcopy(o_a.state_dict())
    o_b.load_offload_state_dict(sd)
    with torch.no_grad():
        for p, q in zip(m_a.parameters(), m_b.parameters()):
            q.copy_(p)
    one_step(m_a, o_a, batches[6:8])
    one_step(m_b, o_b, batches[6:8])
    o_a.synchronize()
    o_b.synchronize()
    same(m_a, o_a, m_b, o_b)


# ------------------------------------------------- resident state vs streamed state
@pytest.mark.gpu
@pytest.mark.parametrize("clip", [None, 0.05])
@pytest.mark.parametrize("staging", [1 << 20, 300 * 1024, 0])
def test_resident_state_equals_streamed_state(clip, staging):
    """Tensors whose state stays in the staging buffer (all of them, some of them, none)
    must step to the same bits as tensors that are loaded every step, and the host copy
    must be current after every step."""
    device = "cuda"
    batches = data(8, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=clip, keep_resident=False, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=clip, staging_bytes=staging, **KW)
    n_res = len(o_b._resident)
    assert not o_a._resident
    if staging == 1 << 20:
        assert n_res == 4            # 4 x 128 x 128 x 8 B = 512 KiB of state fits
    elif staging == 0:
        assert n_res == 0
    else:
        assert n_res == 2            # the last two tensors stay, the first two stream
    for s in range(4):
        one_step(m_a, o_a, batches[2 * s:2 * s + 2])
        one_step(m_b, o_b, batches[2 * s:2 * s + 2])
        if s == 1:
            o_b.wait_writeback()
            o_a.wait_writeback()
            torch.cuda.current_stream().synchronize()
            same(m_a, o_a, m_b, o_b)
    o_a.synchronize()
    o_b.synchronize()
    same(m_a, o_a, m_b, o_b)
    h2d_a, _ = o_a._engine.bytes_moved()
    h2d_b, _ = o_b._engine.bytes_moved()
    if n_res == 4:
        assert h2d_b * 3 < h2d_a  # loaded once instead of four times


@pytest.mark.gpu
@pytest.mark.parametrize("staging", [1 << 20, 300 * 1024])
def test_on_demand_writeback_of_resident_state(staging):
    """``resident_writeback='on_demand'``: resident state stays on the GPU between steps
    (no write-back traffic for it), the host copy is made current by ``wait_writeback()``,
    ``state_dict()`` and a resume, and every step computes the same bits as with a
    write-back per step."""
    device = "cuda"
    batches = data(10, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=0.05, staging_bytes=staging, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=0.05, staging_bytes=staging, resident_writeback="on_demand", **KW)
    assert len(o_a._resident) == len(o_b._resident) > 0
    for s in range(3):
        one_step(m_a, o_a, batches[2 * s:2 * s + 2])
        one_step(m_b, o_b, batches[2 * s:2 * s + 2])
    torch.cuda.synchronize()
    _, d2h_a = o_a._engine.bytes_moved()
    _, d2h_b = o_b._engine.bytes_moved()
    assert d2h_b < d2h_a
    o_a.wait_writeback()
    o_b.wait_writeback()       # the resident tensors go back now, once
    same(m_a, o_a, m_b, o_b)
    _, d2h_b2 = o_b._engine.bytes_moved()
    assert d2h_b2 > d2h_b and d2h_b2 < d2h_a
    # a state_dict() in the middle of training and a resume into the lazy optimizer
    one_step(m_a, o_a, batches[6:8])
    one_step(m_b, o_b, batches[6:8])
    sd_a, sd_b = o_a.state_dict(), o_b.state_dict()
    for sa, sb in zip(sd_a["state"].values(), sd_b["state"].values()):
        for k in sa:
            if torch.is_tensor(sa[k]):
                assert torch.equal(sa[k].cpu(), sb[k].cpu()), k
    o_b.load_offload_state_dict(copy.deepcopy(sd_a))
    one_step(m_a, o_a, batches[8:10])
    one_step(m_b, o_b, batches[8:10])
    o_a.synchronize()
    o_b.synchronize()
    same(m_a, o_a, m_b, o_b)


def test_unknown_resident_writeback_is_rejected():
    with pytest.raises(ValueError, match="resident_writeback"):
        OffloadAdam(net("cpu"), resident_writeback="never", **KW)


@pytest.mark.gpu
def test_resume_reloads_resident_state():
    device = "cuda"
    batches = data(8, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=1.0, staging_bytes=1 << 20, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=1.0, staging_bytes=1 << 20, **KW)
    assert len(o_b._resident) == 4
    one_step(m_a, o_a, batches[0:2])
    one_step(m_a, o_a, batches[2:4])
    one_step(m_b, o_b, batches[4:6])
    sd = copy.deepcopy(o_a.state_dict())
    o_b.load_offload_state_dict(sd)   # the resident copies of B are stale now
    with torch.no_grad():
        for p, q in zip(m_a.parameters(), m_b.parameters()):
            q.copy_(p)
    one_step(m_a, o_a, batches[6:8])
    one_step(m_b, o_b, batches[6:8])
    o_a.synchronize()
    o_b.synchronize()
    same(m_a, o_a, m_b, o_b)


@pytest.mark.gpu
@pytest.mark.parametrize("staging", [1 << 20, 0])
def test_guard_words_stay_intact_and_do_not_change_results(staging):
    """``debug_canaries=True`` puts a guard behind every staging chunk and resident tensor and
    verifies it after each step kernel: the kernels must leave them intact (``synchronize()``
    would raise), and the run must equal one without guards bit for bit.  That an overwritten
    guard is reported is tested against the stand-in runtime (tests/native/engine_stress.cpp)."""
    device = "cuda"
    batches = data(8, device)
    m_a, m_b = net(device), net(device)
    o_a = OffloadAdam(m_a, max_grad_norm=0.05, staging_bytes=staging, **KW)
    o_b = OffloadAdam(m_b, max_grad_norm=0.05, staging_bytes=staging, debug_canaries=True, **KW)
    for s in range(4):
        one_step(m_a, o_a, batches[2 * s:2 * s + 2])
        one_step(m_b, o_b, batches[2 * s:2 * s + 2])
    o_a.synchronize()
    o_b.synchronize()
    same(m_a, o_a, m_b, o_b)
