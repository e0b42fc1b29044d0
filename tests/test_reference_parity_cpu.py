"""Parity with the reference package itself, on CPU, when it is installed under
``baseline/_ref`` (skipped otherwise): what its weight formats write to a checkpoint
must equal what ours write, bit for bit, for the same weights; each side must load the
other's checkpoint; the HF quantization configs must be the same dicts; and one step
of its Adam kernels, run by Triton's interpreter from the same non-trivial state, must
give our high-precision parameter to fp32 rounding and our bf16 moments to one unit in
the last place (the interpreter evaluates scalar expressions in double precision and
truncates fp32 to bf16 where the GPU rounds to nearest even, so more is not expected)."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "offload_adam")),
                                reason="reference package not installed under baseline/_ref")

FORMATS = [("NVFP4QWeight", {}), ("NF4QWeight", {"blocksize": 64}), ("Int4QWeight", {"group_size": 128}),
           ("Int8QWeight", {})]


@pytest.fixture(scope="module")
def ref_qweight():
    sys.path.insert(0, REF)
    try:
        import offload_adam.qweight as rq
    except Exception as e:  # e.g. a Triton build that cannot be imported here
        pytest.skip(f"reference package cannot be imported: {e}")
    finally:
        sys.path.remove(REF)
    return rq


def bits(t):
    return t.view(torch.uint8) if t.element_size() == 1 else t


def weights(shape, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(*shape, generator=g) * 0.05).to(torch.bfloat16)
    x[3, 5] = 1.25   # an outlier that sets the tensor-wide scale
    x[7, :16] = 0.0  # an all-zero block
    return x


@pytest.mark.parametrize("name,kw", FORMATS)
@pytest.mark.parametrize("shape", [(64, 256), (40, 256), (128, 384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_checkpoint_tensors_are_bit_identical(ref_qweight, name, kw, shape, dtype):
    import offload_adam_b200.qweight as oq
    x = weights(shape, seed=shape[0])
    if dtype is torch.float32:  # what an fp32 master looks like: not representable in bf16
        x = x.float() * (1.0 + 1e-3 * torch.sin(torch.arange(x.numel()).float()).reshape(x.shape))
    theirs = getattr(ref_qweight, name).from_float(x, **kw)
    ours = getattr(oq, name).from_float(x, **kw)
    tp, op = theirs.to_plain_state_dict(), ours.to_plain_state_dict()
    assert sorted(tp) == sorted(op)
    assert tuple(getattr(ref_qweight, name).canonical_key_suffixes()) == tuple(getattr(oq, name).canonical_key_suffixes())
    for k in tp:
        assert tp[k].dtype == op[k].dtype and tp[k].shape == op[k].shape, k
        assert torch.equal(bits(tp[k]), bits(op[k])), k
    # each side loads the other's checkpoint and ends with the packed weight the reference
    # gets from its own file (NVFP4 stores the reciprocal of the tensor scale, so a reload
    # is not the identity on that scalar for either implementation)
    t_reload = getattr(ref_qweight, name).from_plain_state_dict(tp, reference=theirs)
    o_cross = getattr(oq, name).from_plain_state_dict(tp, reference=ours)
    t_cross = getattr(ref_qweight, name).from_plain_state_dict(op, reference=theirs)
    for attr in getattr(oq, name).PAYLOAD:
        want = getattr(t_reload, attr)
        assert torch.equal(bits(getattr(o_cross, attr)), bits(want)), attr
        assert torch.equal(bits(getattr(t_cross, attr)), bits(want)), attr


def test_dequantization_matches_the_reference_python_paths(ref_qweight):
    import offload_adam_b200.qweight as oq
    from offload_adam.qweight import int8 as r_int8, nf4 as r_nf4, nvfp4 as r_nvfp4
    x = weights((64, 256), seed=9)
    t, o = ref_qweight.NVFP4QWeight.from_float(x), oq.NVFP4QWeight.from_float(x)
    for dt in (torch.float32, torch.bfloat16):
        want = r_nvfp4.dequantize_nvfp4_blockwise(t.weight_packed, t.block_scale_fp8, t.global_scale, 256, dtype=dt)
        assert torch.equal(o.dequantize(dt), want)
    t, o = ref_qweight.NF4QWeight.from_float(x), oq.NF4QWeight.from_float(x)
    want = r_nf4.dequantize_nf4_blockwise(t.weight_packed, t.absmax, 256, 64, dtype=torch.float32)
    assert torch.equal(o.dequantize(torch.float32), want)
    t, o = ref_qweight.Int8QWeight.from_float(x), oq.Int8QWeight.from_float(x)
    assert torch.equal(o.dequantize(), r_int8.dequantize_int8_per_channel(t.weight, t.scales))
    assert torch.equal(o.dequantize(torch.float32), t.dequantize(torch.float32))  # python fallback of the reference
    t, o = ref_qweight.Int4QWeight.from_float(x, group_size=128), oq.Int4QWeight.from_float(x, group_size=128)
    assert torch.equal(o.dequantize(torch.float32), t.dequantize(torch.float32))  # python fallback of the reference


@pytest.mark.parametrize("name,kw", FORMATS)
def test_hf_quantization_configs_are_the_same_dicts(ref_qweight, name, kw):
    import offload_adam_b200.qweight as oq
    kw = {k: v for k, v in kw.items() if k == "group_size"}
    theirs = getattr(ref_qweight, name).build_hf_quantization_config(skip_patterns=("lm_head",), **kw)
    ours = getattr(oq, name).build_hf_quantization_config(skip_patterns=("lm_head",), **kw)
    assert theirs == ours


STEP_SCRIPT = textwrap.dedent("""
    import os, sys
    os.environ["TRITON_INTERPRET"] = "1"
    import torch, triton
    sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
    from offload_adam.kernels import fp32_master as rf, fp31_master as r31, fp32_master_custom_rounding as rc
    from offload_adam_b200.ops import oracle
    from offload_adam_b200.ops.adam_step import adam_step

    def bh(b, t):
        return (b ** t - b) / (b ** t - 1)

    for mode in ("fp32_master", "fp31_master", "fp32_master_custom_rounding"):
        for decoupled in (True, False):
            n, B = 4096 + 37, 1024
            torch.manual_seed(1)
            p0 = (torch.randn(n) * 0.05).to(torch.bfloat16)
            g = (torch.randn(n) * 1e-2).to(torch.bfloat16)
            m0 = (torch.randn(n) * 1e-2).to(torch.bfloat16)
            v0 = (torch.rand(n) * 1e-4).to(torch.bfloat16)

            def fresh():
                st = {"exp_avg": m0.clone(), "exp_avg_sq": v0.clone()}
                if mode == "fp32_master":
                    st["master_params"] = p0.float() + 1e-4 * torch.sin(torch.arange(n).float())
                else:
                    st["rounding_error"] = ((torch.arange(n) * 37) % 20011 - 10000).to(torch.int16)
                return p0.clone(), st

            pr, sr = fresh()
            po, so = fresh()
            t = 5
            grid = (triton.cdiv(n, B),)
            args = (1e-3, 0.01, bh(0.9, t), bh(0.999, t), 1e-8, n, decoupled, B)
            if mode == "fp32_master":
                rf.adam_step_fp32_master_kernel[grid](pr, g, sr["exp_avg"], sr["exp_avg_sq"], sr["master_params"], *args)
            elif mode == "fp31_master":
                r31.adam_step_fp31_master_kernel[grid](pr, g, sr["exp_avg"], sr["exp_avg_sq"], sr["rounding_error"], *args)
            else:
                rc.adam_step_fp32_master_custom_rounding_kernel[grid](pr, g, sr["exp_avg"], sr["exp_avg_sq"], sr["rounding_error"], *args)
            mine = dict(so)
            mine["grad"] = g
            adam_step(mode, po, mine, 1e-3, 0.01, 0.9, 0.999, 1e-8, t, decoupled_weight_decay=decoupled)
            if mode == "fp32_master":
                ma, mb = sr["master_params"], so["master_params"]
            elif mode == "fp31_master":
                ma, mb = oracle.fp31_reconstruct(pr, sr["rounding_error"]), oracle.fp31_reconstruct(po, so["rounding_error"])
            else:
                ma, mb = oracle.custom_reconstruct(pr, sr["rounding_error"]), oracle.custom_reconstruct(po, so["rounding_error"])
            # the high-precision parameter never passes through a bf16 cast: it must agree to
            # fp32 rounding (2 units of the dropped bit for the 31-bit mode)
            tol = 4e-7 if mode != "fp31_master" else 8e-7
            rel = float(((ma - mb).abs() / mb.abs().clamp(min=1e-3)).max())
            assert rel < tol, (mode, decoupled, rel)
            # moments: bf16 outputs, within one unit in the last place of each other
            for k in ("exp_avg", "exp_avg_sq"):
                a, b = sr[k].float(), so[k].float()
                big = torch.maximum(a.abs(), b.abs())
                ulp = big.clamp(min=2.0 ** -100).log2().floor().exp2() * 2.0 ** -7
                ok = ((a - b).abs() <= ulp) | (big < 1e-6)  # cancellation near zero aside
                assert bool(ok.all()), (mode, k, int((~ok).sum()))
    # the stochastic-rounding rule is integer arithmetic: exact for any random word
    import triton.language as tl
    from offload_adam.kernels import stochastic_rounding as rsr

    @triton.jit
    def sr_kernel(x_ptr, r_ptr, o_ptr, n, B: tl.constexpr):
        offs = tl.program_id(0) * B + tl.arange(0, B)
        mask = offs < n
        x = tl.load(x_ptr + offs, mask=mask)
        r = tl.load(r_ptr + offs, mask=mask)
        tl.store(o_ptr + offs, rsr._fp32_to_bf16_sr(x, r), mask=mask)

    n = 5000
    x = torch.randn(n) * torch.logspace(-6, 3, n)
    x[:6] = torch.tensor([0.0, -0.0, 1.0, -1.0, 1.00390625, -3.0e38])
    r = torch.randint(0, 1 << 16, (n,), dtype=torch.int32)
    r[:6] = torch.tensor([0, 0xFFFF, 0, 0xFFFF, 0x7FFF, 0])
    out = torch.empty(n, dtype=torch.bfloat16)
    sr_kernel[(triton.cdiv(n, 1024),)](x, r, out, n, 1024)
    assert torch.equal(out, oracle.bf16_sr(x, r)), "stochastic rounding rule differs"
    print("OK")
""")


@pytest.mark.timeout(900)
def test_one_adam_step_of_the_reference_kernels_agrees(tmp_path):
    script = tmp_path / "step_parity.py"
    script.write_text(STEP_SCRIPT)
    run = subprocess.run([sys.executable, str(script), REF, ROOT], capture_output=True, text=True, timeout=850)
    if run.returncode != 0 and ("active drivers" in run.stderr or "No module named 'triton'" in run.stderr):
        pytest.skip("Triton's interpreter is not usable here")
    assert run.returncode == 0 and "OK" in run.stdout, run.stderr[-3000:]


class TwoLinears(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = torch.nn.Linear(256, 256, bias=False)
        self.l2 = torch.nn.Linear(256, 128, bias=True)
        self.lm_head = torch.nn.Linear(128, 64, bias=False)

    def forward(self, x):
        return self.lm_head(self.l2(torch.relu(self.l1(x))))


@pytest.mark.parametrize("name,kw", FORMATS)
def test_model_state_dicts_are_interchangeable(ref_qweight, name, kw):
    """``quantize_linears`` + ``model.state_dict()``: same keys, same bits, and each
    package loads the other's state dict into its own quantized model."""
    import offload_adam_b200.qweight as oq
    kw = {k: v for k, v in kw.items() if k in ("group_size", "blocksize")}

    def fresh():
        torch.manual_seed(3)
        return TwoLinears().to(torch.bfloat16)

    theirs, ours = fresh(), fresh()
    ref_qweight.quantize_linears(theirs, getattr(ref_qweight, name), skip_patterns=("lm_head",), **kw)
    oq.quantize_linears(ours, getattr(oq, name), skip_patterns=("lm_head",), **kw)
    ts, os_ = theirs.state_dict(), ours.state_dict()
    assert list(ts) == list(os_)
    for k in ts:
        assert type(ts[k]) is torch.Tensor and type(os_[k]) is torch.Tensor, k
        assert ts[k].dtype == os_[k].dtype and ts[k].shape == os_[k].shape, k
        assert torch.equal(bits(ts[k]), bits(os_[k])), k
    # cross-loading: a differently initialised quantized model takes the other package's file
    torch.manual_seed(11)
    other_ours = TwoLinears().to(torch.bfloat16)
    oq.quantize_linears(other_ours, getattr(oq, name), skip_patterns=("lm_head",), **kw)
    other_ours.load_state_dict(ts)
    torch.manual_seed(12)
    other_theirs = TwoLinears().to(torch.bfloat16)
    ref_qweight.quantize_linears(other_theirs, getattr(ref_qweight, name), skip_patterns=("lm_head",), **kw)
    other_theirs.load_state_dict(os_)
    a, b = other_ours.state_dict(), other_theirs.state_dict()
    reload_theirs = fresh()
    ref_qweight.quantize_linears(reload_theirs, getattr(ref_qweight, name), skip_patterns=("lm_head",), **kw)
    reload_theirs.load_state_dict(ts)
    want = reload_theirs.state_dict()  # what the reference has after reading its own file
    for k in want:
        assert torch.equal(bits(a[k]), bits(want[k])), k
        assert torch.equal(bits(b[k]), bits(want[k])), k
