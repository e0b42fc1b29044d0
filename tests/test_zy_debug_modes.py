"""Debugging aids and host-state hand-offs of the offloaded optimizer: the serialized
mode against the overlapped run, NVTX ranges, waiting for write-backs, and resuming
into an optimizer that has already loaded state for its next step ahead of time; and the
fake-quantization helper."""

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


# ---------------------------------------------------------------- fake quantization
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("fmt", ["nvfp4", "nf4", "int4", "int8"])
def test_fake_quantize_is_quantize_then_dequantize_with_straight_through_gradient(fmt, device):
    from offload_adam_b200.qweight import (Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight,
                                           fake_quantize)
    cls = {"nvfp4": NVFP4QWeight, "nf4": NF4QWeight, "int4": Int4QWeight, "int8": Int8QWeight}[fmt]
    torch.manual_seed(2)
    x = (torch.randn(64, 256, device=device) * 0.05).to(torch.bfloat16).requires_grad_(True)
    y = fake_quantize(x, cls)
    q = cls.from_float(torch.zeros(64, 256, dtype=torch.bfloat16, device=device))
    q.copy_(x.detach().float() if device == "cuda" else x.detach())
    assert y.dtype == x.dtype and torch.equal(y, q.dequantize(torch.bfloat16))
    err = (y.float() - x.detach().float()).abs().max().item()
    assert 0 < err < 0.05
    (y.float() * 2).sum().backward()
    assert torch.equal(x.grad, torch.full_like(x, 2.0))
    with pytest.raises(ValueError):
        fake_quantize(torch.randn(4, 7, device=device).to(torch.bfloat16), cls)
