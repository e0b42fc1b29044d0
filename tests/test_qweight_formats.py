"""Quantized weight formats: storage layout anchors, PyTorch restatement properties,
autograd through F.linear, re-quantization by copy_, and (on a GPU) bit parity of the
sm_100a quantize / dequantize kernels with the restatements."""

import pytest
import torch
import torch.nn.functional as F

from offload_adam_b200.qweight import Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight
from offload_adam_b200.qweight import int4, int8, nf4, nvfp4

FORMATS = [
    (NVFP4QWeight, {}),
    (NF4QWeight, {"blocksize": 64}),
    (Int4QWeight, {"group_size": 128}),
    (Int8QWeight, {}),
]
IDS = ["nvfp4", "nf4", "int4", "int8"]


def payload_equal(a, b):
    return all(torch.equal(x.view(torch.uint8) if x.dtype == torch.float8_e4m3fn else x,
                           y.view(torch.uint8) if y.dtype == torch.float8_e4m3fn else y)
               for x, y in zip(a._payload(), b._payload()))


# ------------------------------------------------------------------ layouts
def test_fp4_pack_layout_and_lut():
    codes = torch.tensor([[1, 2, 3, 4], [15, 0, 8, 7]], dtype=torch.uint8)
    packed = nvfp4.pack_fp4(codes)
    assert packed.tolist() == [[0x21, 0x43], [0x0F, 0x78]]  # even column in the low nibble
    assert torch.equal(nvfp4.unpack_fp4(packed), codes)
    lut = nvfp4.FP4_E2M1_LUT
    assert len(lut) == 16 and lut[:8] == (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
    assert all(lut[i + 8] == -lut[i] for i in range(8))


def test_nf4_pack_layout_and_lut():
    idx = torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8)
    packed = nf4.pack_nf4(idx)
    assert packed.tolist() == [[0x12, 0x34]]  # even column in the HIGH nibble
    assert torch.equal(nf4.unpack_nf4(packed), idx)
    lut = nf4.NF4_LUT
    assert len(lut) == 16 and lut[0] == -1.0 and lut[7] == 0.0 and lut[15] == 1.0
    assert all(a < b for a, b in zip(lut, lut[1:]))


def test_int4_gptq_layout_anchor():
    vals = torch.tensor([[-8, -7, -6, -5, 0, 1, 6, 7], [7, 7, 7, 7, 7, 7, 7, 7]], dtype=torch.int8)
    packed = int4.pack_int4_gptq(vals)
    assert packed.shape == (1, 2) and packed.dtype == torch.int32
    # nibbles (v + 8), least significant first: 0,1,2,3,8,9,14,15
    assert packed[0, 0].item() & 0xFFFFFFFF == 0xFE983210
    assert packed[0, 1].item() & 0xFFFFFFFF == 0xFFFFFFFF
    assert torch.equal(int4.unpack_int4_gptq(packed), vals)


def test_int8_rails_and_scale_anchor():
    w = torch.tensor([[-2.0, 1.0, 2.0, 0.0], [0.5, -0.25, 0.0, 0.125]])
    q, s = int8.quantize_int8_per_channel(w)
    assert q[0].tolist() == [-127, 64, 127, 0]  # 63.5 rounds half to even
    assert torch.allclose(s, torch.tensor([2.0 / 127, 0.5 / 127]))
    assert q.dtype == torch.int8 and q.abs().max() <= 127


def test_e2m1_rounding_every_midpoint():
    """Ties go to the code with an even mantissa; just off a tie goes to the nearer code."""
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i in range(7):
        mid = (mags[i] + mags[i + 1]) / 2
        lo_code, hi_code = i, i + 1
        tie_code = lo_code if lo_code % 2 == 0 else hi_code
        x = torch.tensor([mid, mid * (1 - 1e-6), mid * (1 + 1e-6), -mid], dtype=torch.float32)
        got = nvfp4._quantize_fp4_e2m1_rne(x).tolist()
        assert got == [tie_code, lo_code, hi_code, tie_code | 8], (i, got)
    sat = nvfp4._quantize_fp4_e2m1_rne(torch.tensor([100.0, -100.0, 0.0, -0.0]))
    assert sat.tolist() == [7, 15, 0, 8]


def test_nvfp4_decode_all_codes():
    packed = torch.arange(256, dtype=torch.uint8).reshape(32, 8)
    scale = torch.ones(32, 1).to(torch.float8_e4m3fn)
    out = nvfp4.dequantize_nvfp4_blockwise(packed, scale, torch.tensor(1.0), 16)
    lut = torch.tensor(nvfp4.FP4_E2M1_LUT)
    flat = torch.arange(256)
    assert torch.equal(out[:, 0::2].reshape(-1), lut[flat & 15])
    assert torch.equal(out[:, 1::2].reshape(-1), lut[flat >> 4])
    assert torch.signbit(out[:, 0::2].reshape(-1)[8])  # code 8 is -0.0


# -------------------------------------------------- restatement-level behaviour
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_quantize_shapes_and_error(cls, kw):
    torch.manual_seed(0)
    w = torch.randn(48, 256).to(torch.bfloat16)
    q = cls.from_float(w, **kw)
    assert q.shape == w.shape and q.dtype == torch.bfloat16 and isinstance(q, cls)
    err = (q.dequantize().float() - w.float()).abs().max().item()
    bound = {"nvfp4": 1.2, "nf4": 0.8, "int4": 0.6, "int8": 0.03}[IDS[[c for c, _ in FORMATS].index(cls)]]
    assert err < bound
    assert cls.can_quantize(w, **kw)
    assert not cls.can_quantize(torch.randn(4, 10), **kw)
    assert not cls.can_quantize(torch.randn(256), **kw)


@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_linear_autograd_matches_dense(cls, kw):
    torch.manual_seed(1)
    w = torch.randn(32, 256).to(torch.bfloat16)
    q = torch.nn.Parameter(cls.from_float(w, **kw))
    dense = q.data.dequantize(torch.float32).clone().requires_grad_(True)
    x1 = torch.randn(3, 5, 256, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_(True)
    b = torch.randn(32)
    F.linear(x1, q, b).pow(2).sum().backward()
    F.linear(x2, dense, b).pow(2).sum().backward()
    assert type(q.grad) is torch.Tensor and q.grad.shape == w.shape
    assert torch.allclose(q.grad.float(), dense.grad, rtol=1e-2, atol=1e-2)  # grad is cast to the bf16 outer dtype
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_copy_requantizes_and_tensor_ops(cls, kw):
    torch.manual_seed(2)
    w = torch.randn(32, 256).to(torch.bfloat16)
    q = cls.from_float(w, **kw)
    new = torch.randn(32, 256)
    q.copy_(new)
    assert payload_equal(q, cls.from_float(new, **kw))
    c = q.clone()
    assert isinstance(c, cls) and payload_equal(c, q) and c._payload()[0].data_ptr() != q._payload()[0].data_ptr()
    assert isinstance(q.detach(), cls)
    assert q.to(torch.float16).dtype == torch.float16
    z = torch.zeros_like(q)
    assert type(z) is torch.Tensor and z.shape == q.shape and z.dtype == q.dtype
    dst = torch.empty(32, 256)
    dst.copy_(q)
    assert torch.equal(dst, q.dequantize().float())
    q2 = cls.from_float(w, **kw)
    q2.copy_(q)
    assert payload_equal(q2, q)
    with pytest.raises(NotImplementedError):
        torch.ops.aten.add.Tensor(q, q)


# --------------------------------------------------------------------- GPU
SHAPES = [(32, 256), (35, 256), (128, 1024), (64, 128), (257, 512)]


@pytest.mark.gpu
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_gpu_quantize_kernel_bit_parity(cls, kw, shape, dtype):
    torch.manual_seed(shape[0])
    src = (torch.randn(shape) * 0.1).to(dtype).cuda()
    src[0, :16] = 0  # an all-zero block
    src[1, 3] = 7.5  # an outlier setting the tensor amax
    outer = torch.bfloat16 if dtype == torch.float32 else dtype
    # destination allocated through the restatement, then overwritten by the kernel
    dst = cls.from_float(torch.zeros(shape, dtype=outer, device="cuda"), **kw)
    dst.copy_(src)  # kernel path
    host = cls.from_float(torch.zeros(shape, dtype=outer), **kw)
    host.copy_(src.cpu())  # restatement path
    for a, b in zip(dst._payload(), host._payload()):
        a, b = a.cpu(), b
        if a.dtype == torch.float8_e4m3fn:
            a, b = a.view(torch.uint8), b.view(torch.uint8)
        assert torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_gpu_dequantize_kernel_bit_parity(cls, kw, shape, dtype):
    torch.manual_seed(shape[1])
    w = (torch.randn(shape) * 0.3).to(torch.bfloat16 if dtype == torch.float32 else dtype)
    if cls in (Int4QWeight, Int8QWeight):
        if dtype == torch.float32:
            pytest.skip("int formats dequantize in their scale dtype")
        q = cls.from_float(w, scale_dtype=dtype, **kw)
    else:
        q = cls.from_float(w, **kw)
    want = q.dequantize(dtype)
    got = q.to("cuda").dequantize(dtype)
    assert got.is_cuda and got.dtype == want.dtype
    assert torch.equal(got.cpu().view(torch.int16 if dtype != torch.float32 else torch.int32),
                       want.view(torch.int16 if dtype != torch.float32 else torch.int32))


@pytest.mark.gpu
def test_gpu_nvfp4_all_scale_bytes_and_codes():
    """Every e4m3 encoding (NaN excluded) and every FP4 code through the kernel."""
    packed = torch.arange(256, dtype=torch.uint8).repeat_interleave(8).reshape(256, 8)
    scale_bytes = torch.arange(256, dtype=torch.uint8)
    keep = (scale_bytes & 0x7F) != 0x7F
    packed, scale_bytes = packed[keep], scale_bytes[keep]
    scale = scale_bytes.view(torch.float8_e4m3fn).reshape(-1, 1)
    g = torch.tensor(0.37)
    want = nvfp4.dequantize_nvfp4_blockwise(packed, scale, g, 16, torch.float32)
    got = nvfp4._dequant_nvfp4_cuda(packed.cuda(), scale.cuda(), g.cuda(), 16, torch.float32)
    assert torch.equal(got.cpu().view(torch.int32), want.view(torch.int32))


@pytest.mark.gpu
def test_gpu_nvfp4_quantize_stress_with_boundaries():
    torch.manual_seed(7)
    n = 1 << 20
    x = torch.randn(n) * 2
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    # plant exact midpoints (relative to a block whose amax maps to 6) and signed zeros
    x[:7] = mids
    x[7:14] = -mids
    x[14], x[15] = 6.0, -0.0
    x = x.reshape(1024, 1024)
    p_ref, s_ref, g_ref = nvfp4.quantize_nvfp4_blockwise(x)
    p, s, g = nvfp4._quantize_nvfp4_cuda(x.cuda())
    assert torch.equal(g.cpu(), g_ref)
    assert torch.equal(s.cpu().view(torch.uint8), s_ref.view(torch.uint8))
    assert torch.equal(p.cpu(), p_ref)
    # amax supplied by the caller (as the fused optimizer step does) gives the same bytes
    amax = x.abs().max().reshape(1).cuda()
    p2, s2, g2 = nvfp4._quantize_nvfp4_cuda(x.cuda(), amax=amax)
    assert torch.equal(p2, p) and torch.equal(g2, g)


@pytest.mark.gpu
def test_gpu_nf4_ties_pick_lowest_index():
    lut = torch.tensor(nf4.NF4_LUT)
    mids = (lut[:-1] + lut[1:]) / 2
    x = torch.zeros(2, 64)
    x[0, :15] = mids
    x[0, 63] = 1.0  # absmax 1 keeps the midpoints unscaled
    x[1, :15] = -mids.flip(0)
    x[1, 63] = -1.0
    p_ref, a_ref = nf4.quantize_nf4_blockwise(x, 64)
    p, a = nf4._quantize_nf4_cuda(x.cuda(), 64)
    assert torch.equal(p.cpu(), p_ref) and torch.equal(a.cpu(), a_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_gpu_linear_and_requantize(cls, kw):
    torch.manual_seed(3)
    w = (torch.randn(64, 256) * 0.1).to(torch.bfloat16).cuda()
    q = torch.nn.Parameter(cls.from_float(w, **kw))
    x = torch.randn(8, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    F.linear(x, q).float().pow(2).mean().backward()
    assert q.grad is not None and type(q.grad) is torch.Tensor and x.grad is not None
    master = w.float() * 0.5
    q.data.copy_(master)
    assert torch.allclose(q.data.dequantize().float(), master, atol=0.15)


# --------------------------------------------------------------- row shards
def _same_bits(a, b):
    a = a.view(torch.uint8) if a.element_size() == 1 else a
    b = b.view(torch.uint8) if b.element_size() == 1 else b
    return torch.equal(a, b)


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
@pytest.mark.parametrize("fmt", ["nvfp4", "nf4", "int4", "int8"])
def test_row_shards_requantize_to_the_same_bits(fmt, device):
    """Quantizing row ranges separately (as the owners of a sharded weight do) must
    reproduce the whole-tensor quantization bit for bit."""
    from offload_adam_b200.qweight import Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight
    cls = {"nvfp4": NVFP4QWeight, "nf4": NF4QWeight, "int4": Int4QWeight, "int8": Int8QWeight}[fmt]
    torch.manual_seed(1)
    master = (torch.randn(256, 384, device=device) * 0.05)
    master[200, 7] = 1.5  # the tensor-wide maximum sits in the last shard
    whole = cls.from_float(torch.zeros(256, 384, dtype=torch.bfloat16, device=device))
    whole.copy_(master)
    split = cls.from_float(torch.zeros(256, 384, dtype=torch.bfloat16, device=device))
    amax = master.abs().amax().reshape(1).float() if cls.USES_TENSOR_AMAX else None
    for lo, hi in ((0, 64), (64, 128), (128, 256)):
        shard, views = split.row_shard(lo, hi)
        assert tuple(shard.shape) == (hi - lo, 384)
        shard._quantize_into(master[lo:hi].contiguous(), amax)
        for view, part in zip(views, shard._payload()):
            if part.data_ptr() != view.data_ptr():
                view.copy_(part)
    for a, b in zip(whole._payload(), split._payload()):
        assert _same_bits(a, b)


# ---------------------------------------------------------------- fake quantization
@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
@pytest.mark.parametrize("fmt", ["nvfp4", "nf4", "int4", "int8"])
def test_fake_quantize_is_quantize_then_dequantize_with_straight_through_gradient(fmt, device):
    from offload_adam_b200.qweight import fake_quantize
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


@pytest.mark.gpu
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
@pytest.mark.parametrize("shape", [(96, 256), (33, 384), (5, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_gpu_one_pass_fake_quantize_equals_quantize_then_dequantize(cls, kw, shape, dtype):
    """The one-pass kernel against the two kernels it replaces, bit for bit."""
    from offload_adam_b200.qweight import fake_quantize
    from offload_adam_b200.qweight.fake_quant import _fake_quantize_cuda
    torch.manual_seed(shape[0] + shape[1])
    x = (torch.randn(shape, device="cuda") * 0.07).to(dtype)
    x[0, :16] = 0
    x[1, 5] = 3.25
    assert _fake_quantize_cuda(x, cls, kw) is not None  # the kernel route takes this case
    y = fake_quantize(x, cls, **kw)
    outer = torch.bfloat16 if dtype == torch.float32 else dtype
    q = cls.from_float(torch.zeros(shape, dtype=outer, device="cuda"), **kw)
    q.copy_(x)
    want = q.dequantize(dtype)
    assert y.dtype == dtype
    bits = torch.int32 if dtype == torch.float32 else torch.int16
    assert torch.equal(y.view(bits), want.view(bits))


# ------------------------------------------ NF4 decision thresholds built into the kernels
def test_nf4_kernel_thresholds_follow_from_the_codebook():
    """The CUDA kernels find the nearest NF4 entry by counting thresholds <= x.  Threshold i is
    the smallest fp32 x for which entry i + 1 is strictly closer than entry i in fp32
    arithmetic; recompute all fifteen by bisection over fp32 values and compare with the
    table in csrc/quant_math.cuh, then check the counting rule against the sequential scan."""
    import os
    import re

    import numpy as np
    lut = np.array(nf4.NF4_LUT, dtype=np.float32)

    def to_ord(x):
        u = int(np.float32(x).view(np.uint32))
        return u + 0x80000000 if u < 0x80000000 else 0xFFFFFFFF - u

    def from_ord(o):
        u = o - 0x80000000 if o >= 0x80000000 else 0xFFFFFFFF - o
        return np.uint32(u).view(np.float32)

    def closer_to_next(x, i):
        x = np.float32(x)
        return abs(np.float32(x - lut[i + 1])) < abs(np.float32(x - lut[i]))

    want = []
    for i in range(15):
        lo, hi = to_ord(lut[i]), to_ord(lut[i + 1])
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if closer_to_next(from_ord(mid), i):
                hi = mid
            else:
                lo = mid
        want.append(int(from_ord(hi).view(np.uint32)))
    header = os.path.join(os.path.dirname(nf4.__file__), "..", "csrc", "quant_math.cuh")
    text = open(header).read()
    block = text[text.index("#define OAB_NF4_THRESHOLD_BITS"):]
    block = block[:block.index("__device__")]
    got = [int(h, 16) for h in re.findall(r"0x([0-9a-fA-F]{8})u", block)]
    assert got == want
    # the counting rule equals the restatement's sequential scan, also next to every threshold
    thr = np.array(want, dtype=np.uint32).view(np.float32)
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.uniform(-1.05, 1.05, 200000).astype(np.float32), thr,
                         np.nextafter(thr, np.float32(-2)), np.nextafter(thr, np.float32(2))])
    count = sum((xs >= t).astype(np.int64) for t in thr)
    best = np.zeros(xs.shape, dtype=np.int64)
    bd = np.full(xs.shape, np.inf, dtype=np.float32)
    for i, v in enumerate(lut):
        d = np.abs((xs - v).astype(np.float32))
        c = d < bd
        best[c] = i
        bd[c] = d[c]
    assert np.array_equal(count, best)
