"""Step of a quantized weight in one pass (``csrc/adam_quant.cu``): Adam on the fp32 master,
re-quantization of the updated rows and the store of the packed rows into every replica.
Checked bit for bit against the separate step kernel followed by the format's PyTorch
quantizer, for a row range inside a larger weight, with two replicas, with a local and
with a pulled (rank-averaged) gradient; and through the optimizers, where chunks of whole
rows stream through a small staging buffer."""

import warnings

import pytest
import torch
import torch.nn as nn

from offload_adam_b200 import Adam, OffloadAdam, _ext
from offload_adam_b200.ops.adam_step import adam_step
from offload_adam_b200.ops.oracle import beta_hat
from offload_adam_b200.qweight import (Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight, int4, int8, nf4,
                                       nvfp4, quantize_linears)

pytestmark = pytest.mark.gpu

HP = dict(lr=1e-2, wd=0.05, b1=0.9, b2=0.999, eps=1e-8, step=3)


def _state(rows, in_f, seed):
    g = torch.Generator().manual_seed(seed)
    master = (torch.randn(rows, in_f, generator=g) * 0.05).cuda()
    grad = (torch.randn(rows, in_f, generator=g) * 0.01).to(torch.bfloat16).cuda()
    m = (torch.randn(rows, in_f, generator=g) * 0.01).to(torch.bfloat16).cuda()
    v = (torch.rand(rows, in_f, generator=g) * 1e-4).to(torch.bfloat16).cuda()
    return master, grad, m, v


def _reference_step(master, grad, m, v, decoupled, clip):
    """The plain step kernel on copies: returns updated (master, m, v)."""
    st = {"grad": grad.clone(), "exp_avg": m.clone(), "exp_avg_sq": v.clone(), "master_params": master.clone()}
    adam_step("fp32_master", None, st, HP["lr"], HP["wd"], HP["b1"], HP["b2"], HP["eps"], HP["step"],
              decoupled_weight_decay=decoupled, clip_coef=clip)
    return st["master_params"], st["exp_avg"], st["exp_avg_sq"]


def _bits(t):
    return t.view(torch.uint8) if t.element_size() == 1 else t


CASES = [
    ("nf4", 64, (96, 256)), ("nf4", 32, (40, 512)), ("nf4", 256, (33, 1024)),
    ("int4", 128, (96, 256)), ("int4", 32, (40, 512)), ("int4", 64, (33, 1024)),
    ("int8", 0, (96, 256)), ("int8", 0, (7, 4096)), ("int8", 0, (33, 1008)),
]


@pytest.mark.parametrize("fmt,group,shape", CASES)
@pytest.mark.parametrize("decoupled", [True, False])
@pytest.mark.parametrize("pulled", [False, True])
def test_fused_step_equals_step_then_quantize(fmt, group, shape, decoupled, pulled):
    C = _ext.load(required=True)
    rows, in_f = shape
    out_f, row0 = rows + 64, 32          # the rows sit inside a larger weight
    master, grad, m, v = _state(rows, in_f, 5 + rows)
    clip = torch.tensor([0.37], device="cuda")
    scale_dtype = torch.bfloat16
    if fmt == "nf4":
        pay = [(torch.zeros(out_f, in_f // 2, dtype=torch.uint8, device="cuda"),
                torch.zeros(out_f * in_f // group, dtype=torch.float32, device="cuda")) for _ in range(2)]
        fid = C.QFMT_NF4
    elif fmt == "int4":
        pay = [(torch.zeros(in_f // 8, out_f, dtype=torch.int32, device="cuda"),
                torch.zeros(in_f // group, out_f, dtype=scale_dtype, device="cuda")) for _ in range(2)]
        fid = C.QFMT_INT4
    else:
        pay = [(torch.zeros(out_f, in_f, dtype=torch.int8, device="cuda"),
                torch.zeros(out_f, dtype=scale_dtype, device="cuda")) for _ in range(2)]
        fid = C.QFMT_INT8
    assert C.adam_quant_supported(fid, in_f, group)
    spec = C.QuantSpec(fid, out_f, in_f, row0, group, C.QDT_BF16, [a.data_ptr() for a, _ in pay],
                       [b.data_ptr() for _, b in pay])
    if pulled:
        # two "ranks" on one device: the gradient is the rank-ordered fp32 mean, rounded once
        g2 = (torch.randn(rows, in_f, device="cuda") * 0.01).to(torch.bfloat16)
        reduced = ((grad.float() + g2.float()) * 0.5).to(torch.bfloat16)
        peers, gscale, garg = [grad.data_ptr(), g2.data_ptr()], 0.5, None
    else:
        reduced, peers, gscale, garg = grad, [], 1.0, grad
    want_master, want_m, want_v = _reference_step(master, reduced, m, v, decoupled, clip)
    C.adam_quant_push(spec, garg, None, m, v, master, HP["lr"], HP["wd"], beta_hat(HP["b1"], HP["step"]),
                      beta_hat(HP["b2"], HP["step"]), HP["eps"], decoupled, clip, 0, 0, peers, gscale, None)
    torch.cuda.synchronize()
    assert torch.equal(master, want_master) and torch.equal(m, want_m) and torch.equal(v, want_v)
    # payload of the updated rows, from the format's PyTorch quantizer
    if fmt == "nf4":
        packed, absmax = nf4.quantize_nf4_blockwise(want_master.cpu(), group)
        per_row = in_f // group
        for a, b in pay:
            assert torch.equal(a[row0:row0 + rows].cpu(), packed)
            assert torch.equal(b[row0 * per_row:(row0 + rows) * per_row].cpu(), absmax)
            assert a[:row0].abs().sum() == 0 and a[row0 + rows:].abs().sum() == 0  # nothing outside the rows
    elif fmt == "int4":
        qw, sc = int4.quantize_int4_groupwise(want_master.cpu(), group, scale_dtype=scale_dtype)
        for a, b in pay:
            assert torch.equal(a[:, row0:row0 + rows].cpu(), qw)
            assert torch.equal(b[:, row0:row0 + rows].cpu(), sc)
            assert a[:, :row0].abs().sum() == 0 and a[:, row0 + rows:].abs().sum() == 0
    else:
        w, sc = int8.quantize_int8_per_channel(want_master.cpu(), scale_dtype=scale_dtype)
        for a, b in pay:
            assert torch.equal(a[row0:row0 + rows].cpu(), w)
            assert torch.equal(b[row0:row0 + rows].cpu(), sc)
            assert a[:row0].abs().sum() == 0 and a[row0 + rows:].abs().sum() == 0


@pytest.mark.parametrize("shape", [(96, 256), (33, 1024), (5, 4096)])
def test_nvfp4_two_pass_step(shape):
    """NVFP4: the step leaves max|master| and a device copy of the master; the second pass
    quantizes with the tensor scale of the WHOLE weight (here larger than the rows' own)."""
    C = _ext.load(required=True)
    rows, in_f = shape
    out_f, row0 = rows + 64, 32
    master, grad, m, v = _state(rows, in_f, 9 + rows)
    want_master, want_m, want_v = _reference_step(master, grad, m, v, True, None)
    amax = torch.zeros(1, device="cuda")
    copy = torch.empty_like(master)
    st = {"grad": grad, "exp_avg": m, "exp_avg_sq": v, "master_params": master}
    C.adam_step(1, None, grad, None, m, v, master, HP["lr"], HP["wd"], beta_hat(HP["b1"], HP["step"]),
                beta_hat(HP["b2"], HP["step"]), HP["eps"], True, None, 0, 0, amax, 0, 0, [], 1.0, [], None, copy)
    torch.cuda.synchronize()
    assert torch.equal(master, want_master) and torch.equal(copy, want_master)
    assert amax.item() == want_master.abs().max().item()
    whole = torch.maximum(amax, torch.tensor([0.9], device="cuda"))  # another rank's rows hold the maximum
    pay = [(torch.zeros(out_f, in_f // 2, dtype=torch.uint8, device="cuda"),
            torch.zeros(out_f, in_f // 16, dtype=torch.uint8, device="cuda")) for _ in range(2)]
    gs = torch.zeros((), device="cuda")
    spec = C.QuantSpec(C.QFMT_NVFP4, out_f, in_f, row0, 16, C.QDT_BF16, [a.data_ptr() for a, _ in pay],
                       [b.data_ptr() for _, b in pay], whole, gs)
    C.nvfp4_quantize_push(spec, copy.data_ptr(), copy.numel(), None, 0)
    torch.cuda.synchronize()
    # the restatement runs on the CPU: a CUDA tensor divided by a Python scalar is multiplied by
    # the scalar's reciprocal, which can differ from the correctly rounded quotient in the last bit
    packed, scale, gscale = nvfp4.quantize_nvfp4_blockwise(want_master.cpu(), amax=whole.cpu())
    assert gs.item() == gscale.item()
    for a, b in pay:
        assert torch.equal(a[row0:row0 + rows].cpu(), packed)
        assert torch.equal(b[row0:row0 + rows].cpu(), scale.view(torch.uint8))
        assert a[:row0].abs().sum() == 0 and a[row0 + rows:].abs().sum() == 0


# ------------------------------------------------------------- through the optimizers
class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(256, 384, bias=False)
        self.l2 = nn.Linear(384, 256, bias=False)
        self.l3 = nn.Linear(256, 128, bias=False)

    def forward(self, x):
        return self.l3(torch.relu(self.l2(torch.relu(self.l1(x)))))


FORMATS = [("nvfp4", NVFP4QWeight, {}), ("nf4", NF4QWeight, {"blocksize": 64}),
           ("int4", Int4QWeight, {"group_size": 128}), ("int8", Int8QWeight, {})]


def _build(cls, kw):
    torch.manual_seed(0)
    m = Block().to(torch.bfloat16).cuda()
    quantize_linears(m, cls, **kw)
    return m


@pytest.mark.parametrize("name,cls,kw", FORMATS, ids=[f[0] for f in FORMATS])
@pytest.mark.parametrize("resident", [False, True])
def test_offloaded_qat_steps_like_the_on_gpu_optimizer(name, cls, kw, resident):
    """OffloadAdam (fused route, chunks of a few rows through a small staging buffer, or
    resident state) must keep packed weights and masters identical to Adam, which steps the
    whole master on the GPU and re-quantizes it with the stand-alone kernels."""
    ma, mb = _build(cls, kw), _build(cls, kw)
    oa = Adam(ma.parameters(), mode="fp32_master", lr=1e-2, weight_decay=0.05, decoupled_weight_decay=True)
    ob = OffloadAdam(mb, mode="fp32_master", lr=1e-2, weight_decay=0.05, decoupled_weight_decay=True,
                     inplace_param_threshold=0, chunk_elems=4096, keep_resident=resident,
                     staging_bytes=(4 << 20) if resident else 0, max_grad_norm=None)
    assert all(ob._fused_quant_plan(p) is not None for p in mb.parameters())
    assert (len(ob._resident) == 3) == resident
    g = torch.Generator().manual_seed(3)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for _ in range(3):
            x = torch.randn(8, 256, generator=g).to(torch.bfloat16).cuda()
            ob.ready_for_optimizer_step = True
            ma(x).float().pow(2).mean().backward()
            mb(x).float().pow(2).mean().backward()
            oa.step()
            ob.step()
            ma.zero_grad(set_to_none=True)
    ob.synchronize()
    for pa, pb in zip(ma.parameters(), mb.parameters()):
        assert torch.equal(oa.state[pa]["master_params"].cpu(), ob.state[pb]["master_params"].cpu())
        assert torch.equal(oa.state[pa]["exp_avg"].cpu(), ob.state[pb]["exp_avg"].cpu())
        for a, b in zip(pa.data._payload(), pb.data._payload()):
            assert torch.equal(_bits(a), _bits(b))


@pytest.mark.parametrize("name,cls,kw", FORMATS, ids=[f[0] for f in FORMATS])
def test_fused_and_unfused_routes_agree_with_clipping(name, cls, kw):
    """Clipping path: the fused route against the unfused one (whole master through a
    device temporary, stand-alone quantize kernel)."""
    ma, mb = _build(cls, kw), _build(cls, kw)
    common = dict(mode="fp32_master", lr=1e-2, weight_decay=0.05, decoupled_weight_decay=True,
                  inplace_param_threshold=0, chunk_elems=4096, max_grad_norm=0.05)
    oa = OffloadAdam(ma, keep_resident=False, **common)
    oa._fused_quant = {p: None for p in ma.parameters()}   # force the unfused route
    ob = OffloadAdam(mb, keep_resident=False, staging_bytes=0, **common)
    g = torch.Generator().manual_seed(4)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for _ in range(3):
            for micro in range(2):
                x = torch.randn(8, 256, generator=g).to(torch.bfloat16).cuda()
                oa.ready_for_optimizer_step = ob.ready_for_optimizer_step = micro == 1
                ma(x).float().pow(2).mean().backward()
                mb(x).float().pow(2).mean().backward()
            oa.step()
            ob.step()
    oa.synchronize()
    ob.synchronize()
    for pa, pb in zip(ma.parameters(), mb.parameters()):
        assert torch.equal(oa.state[pa]["master_params"], ob.state[pb]["master_params"])
        for a, b in zip(pa.data._payload(), pb.data._payload()):
            assert torch.equal(_bits(a), _bits(b))
