"""QAT plumbing around the formats: state_dict hooks, HF quantization configs,
quantize_linears reports, and the optimizer-side contract (fp32 master seeding,
the one-shot lossy-master warning, master refill from checkpoints, resume).

Every scenario runs on CPU; the ``gpu`` variants repeat the optimizer ones on CUDA
with the native kernels and pinned host state."""

import json
import warnings
from types import SimpleNamespace

import pytest
import torch
import torch.nn as nn

from offload_adam_b200 import Adam, OffloadAdam
from offload_adam_b200.qweight import (Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight,
                                       QuantizeReport, quantize_linears, save_quantized_pretrained)

FORMATS = [(Int4QWeight, {"group_size": 128}), (Int8QWeight, {}), (NF4QWeight, {"blocksize": 64}), (NVFP4QWeight, {})]
IDS = ["int4", "int8", "nf4", "nvfp4"]
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


class Block(nn.Module):
    def __init__(self, in_f=256, mid=256, out_f=128):
        super().__init__()
        self.l1 = nn.Linear(in_f, mid, bias=False)
        self.ln = nn.LayerNorm(mid)
        self.l2 = nn.Linear(mid, out_f, bias=True)

    def forward(self, x):
        return self.l2(self.ln(self.l1(x)))


class Two(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(128, 128, bias=False)
        self.l2 = nn.Linear(128, 128, bias=False)

    def forward(self, x):
        return self.l2(self.l1(x))


def build(cls, kw, device="cpu", module=Block):
    torch.manual_seed(0)
    m = module().to(torch.bfloat16).to(device)
    quantize_linears(m, cls, **kw)
    return m


def lossy_warnings(caught):
    return sum("lossy dequant-seeded" in str(w.message) for w in caught)


def save_params(model, path, keys=None):
    from safetensors.torch import save_file
    save_file({n: p.detach().cpu().contiguous() for n, p in model.named_parameters()
               if keys is None or n in keys}, str(path))


# ------------------------------------------------------------ state_dict hooks
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_state_dict_is_plain_and_canonical(cls, kw):
    m = build(cls, kw)
    sd = m.state_dict()
    assert all(type(v) is torch.Tensor for v in sd.values())
    for layer in ("l1", "l2"):
        for suffix in cls.canonical_key_suffixes():
            assert f"{layer}.{suffix}" in sd
    assert {"ln.weight", "ln.bias", "l2.bias"} <= set(sd)


@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_state_dict_round_trips_through_files(cls, kw, tmp_path):
    from safetensors.torch import load_file, save_file
    m = build(cls, kw)
    sd = {k: v.contiguous() for k, v in m.state_dict().items()}
    save_file(sd, str(tmp_path / "m.safetensors"))
    torch.save(sd, tmp_path / "m.pt")
    for loaded in (load_file(str(tmp_path / "m.safetensors")),
                   torch.load(tmp_path / "m.pt", weights_only=True)):
        assert set(loaded) == set(sd)
        fresh = build(cls, kw)
        with torch.no_grad():
            fresh.l1.weight.data.copy_(torch.zeros(256, 256))
        res = fresh.load_state_dict(loaded)
        assert not res.missing_keys and not res.unexpected_keys
        assert isinstance(fresh.l1.weight.data, cls)
        for a, b in zip(fresh.l1.weight.data._payload(), m.l1.weight.data._payload()):
            if a.dtype == torch.float8_e4m3fn:
                a, b = a.view(torch.uint8), b.view(torch.uint8)
            assert torch.equal(a, b)


@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_partial_quant_keys_are_reported_missing(cls, kw):
    m = build(cls, kw)
    sd = m.state_dict()
    dropped = "l1." + cls.canonical_key_suffixes()[-1]
    del sd[dropped]
    res = build(cls, kw).load_state_dict(sd, strict=False)
    assert dropped in res.missing_keys


@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_dense_checkpoint_requantizes_on_load(cls, kw):
    torch.manual_seed(5)
    dense = Block().to(torch.bfloat16)
    m = build(cls, kw)
    res = m.load_state_dict(dense.state_dict())
    assert not res.missing_keys and not res.unexpected_keys
    assert isinstance(m.l1.weight.data, cls)
    want = cls.from_float(dense.l1.weight.data, **kw)
    assert torch.equal(m.l1.weight.data.dequantize(), want.dequantize())


def test_nvfp4_global_scale_is_saved_as_reciprocal():
    m = build(NVFP4QWeight, {})
    sd = m.state_dict()
    g = m.l1.weight.data.global_scale
    assert sd["l1.weight_global_scale"].shape == (1,)
    assert torch.allclose(sd["l1.weight_global_scale"], (1.0 / g).reshape(1))
    with pytest.raises(ValueError, match="reference"):
        NVFP4QWeight.from_plain_state_dict(m.l1.weight.data.to_plain_state_dict())


def test_int8_and_int4_disk_layouts():
    m = build(Int8QWeight, {})
    sd = m.state_dict()
    assert sd["l1.weight_packed"].dtype == torch.int32 and sd["l1.weight_packed"].shape == (256, 64)
    assert sd["l1.weight_scale"].shape == (256, 1) and sd["l1.weight_shape"].tolist() == [256, 256]
    m4 = build(Int4QWeight, {"group_size": 128})
    sd4 = m4.state_dict()
    assert sd4["l1.qweight"].shape == (32, 256) and sd4["l1.scales"].shape == (2, 256)
    assert (sd4["l1.qzeros"] & 0xFFFFFFFF == 0x88888888).all() and sd4["l1.qzeros"].shape == (2, 32)
    nf = build(NF4QWeight, {"blocksize": 64}).state_dict()
    meta = json.loads(bytes(nf["l1.weight.quant_state.bitsandbytes__nf4"].tolist()).decode())
    assert meta == {"quant_type": "nf4", "blocksize": 64, "dtype": "bfloat16", "shape": [256, 256]}
    assert nf["l1.weight"].shape == (256 * 128, 1) and nf["l1.weight.quant_map"].shape == (16,)


# ------------------------------------------------------------------ HF config
def test_hf_quantization_configs():
    c = Int4QWeight.build_hf_quantization_config(skip_patterns=("lm_head",), group_size=128)
    assert c == {"quant_method": "gptq", "bits": 4, "group_size": 128, "desc_act": False, "sym": True,
                 "modules_to_not_convert": ["lm_head"]}
    c = Int8QWeight.build_hf_quantization_config(skip_patterns=("lm_head",))
    assert c["quant_method"] == "compressed-tensors" and c["format"] == "pack-quantized"
    assert c["config_groups"]["group_0"]["weights"] == {"num_bits": 8, "type": "int", "symmetric": True,
                                                        "strategy": "channel"}
    assert c["ignore"] == ["lm_head"]
    c = NF4QWeight.build_hf_quantization_config(skip_patterns=("lm_head",))
    assert c == {"quant_method": "bitsandbytes", "load_in_4bit": True, "bnb_4bit_quant_type": "nf4",
                 "bnb_4bit_use_double_quant": False, "bnb_4bit_compute_dtype": "bfloat16",
                 "llm_int8_skip_modules": ["lm_head"]}
    assert NF4QWeight.build_hf_quantization_config(compute_dtype="float16")["bnb_4bit_compute_dtype"] == "float16"
    c = NVFP4QWeight.build_hf_quantization_config(skip_patterns=("lm_head",))
    w = c["config_groups"]["group_0"]["weights"]
    assert c["format"] == "nvfp4-pack-quantized" and w["num_bits"] == 4 and w["type"] == "float"
    assert w["group_size"] == 16 and w["strategy"] == "tensor_group" and c["ignore"] == ["lm_head"]


def test_update_hf_config_and_save_quantized_pretrained(tmp_path):
    class WithConfig(Two):
        def __init__(self):
            super().__init__()
            self.config = SimpleNamespace()

        def save_pretrained(self, directory):
            directory.mkdir(parents=True, exist_ok=True)
            (directory / "config.json").write_text(json.dumps({"model_type": "fake"}))

    m = WithConfig().to(torch.bfloat16)
    quantize_linears(m, Int4QWeight, group_size=128, skip_patterns=("lm_head",), update_hf_config=True)
    assert m.config.quantization_config["quant_method"] == "gptq"
    m2 = WithConfig().to(torch.bfloat16)
    quantize_linears(m2, Int4QWeight, group_size=128)
    assert not hasattr(m2.config, "quantization_config")
    save_quantized_pretrained(m2, tmp_path / "out", Int4QWeight, skip_patterns=("lm_head",), group_size=128)
    cfg = json.loads((tmp_path / "out" / "config.json").read_text())
    assert cfg["model_type"] == "fake" and cfg["quantization_config"]["modules_to_not_convert"] == ["lm_head"]


# -------------------------------------------------------------- report / strict
def test_quantize_linears_report_and_strict():
    torch.manual_seed(0)
    m = Two().to(torch.bfloat16)
    rep = quantize_linears(m, Int4QWeight, group_size=128, skip_patterns=("l2",))
    assert isinstance(rep, QuantizeReport)
    assert rep.quantized == ["l1"] and rep.excluded == ["l2"] and rep.incompatible == []
    odd = nn.Sequential(nn.Linear(100, 128, bias=False)).to(torch.bfloat16)
    rep = quantize_linears(odd, Int4QWeight, group_size=128)
    assert rep.incompatible and rep.incompatible[0][0] == "0"
    with pytest.raises(ValueError, match="strict=True"):
        quantize_linears(odd, Int4QWeight, group_size=128, strict=True)
    top = nn.Linear(128, 128, bias=False).to(torch.bfloat16)
    quantize_linears(top, Int4QWeight, group_size=128)
    assert "weight" in dict(top.named_parameters())


# ------------------------------------------------------------ optimizer contract
@pytest.mark.parametrize("device", DEVICES)
def test_master_seeding_and_flags(device):
    m = build(Int4QWeight, {"group_size": 128}, device, Two)
    opt = Adam(m.parameters(), mode="fp32_master", lr=1e-3)
    st = opt.state[m.l1.weight]
    opt._init_state_if_empty(m.l1.weight, st)
    assert st["master_filled"] is False
    assert torch.equal(st["master_params"], m.l1.weight.data.dequantize().float())
    dense = Two().to(torch.bfloat16).to(device)
    opt2 = Adam(dense.parameters(), mode="fp32_master")
    st2 = opt2.state[dense.l1.weight]
    opt2._init_state_if_empty(dense.l1.weight, st2)
    assert torch.equal(st2["master_params"], dense.l1.weight.data.float()) and "master_filled" not in st2
    off = OffloadAdam(build(Int4QWeight, {"group_size": 128}, device, Two), mode="fp32_master")
    p = off._offload_params[0]
    assert off.state[p]["master_filled"] is False and off.state[p]["master_params"].dtype == torch.float32
    assert len(off._offload_params) == 2  # quantized params are offloaded whatever their size
    with pytest.raises(ValueError, match="fp32_master"):
        Adam(m.parameters(), mode="stochastic_rounding")
    with pytest.raises(ValueError, match="fp32_master"):
        OffloadAdam(m, mode="fp31_master")


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("kind", ["adam", "offload"])
def test_lossy_master_warns_exactly_once(device, kind):
    m = build(Int4QWeight, {"group_size": 128}, device, Two)
    opt = Adam(m.parameters(), mode="fp32_master", lr=1e-3) if kind == "adam" else \
        OffloadAdam(m, mode="fp32_master", lr=1e-3)
    x = torch.randn(4, 128, dtype=torch.bfloat16, device=device)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        opt.step()  # nothing to step yet: must not consume the warning
    assert lossy_warnings(caught) == 0
    counts = []
    for _ in range(2):
        opt.ready_for_optimizer_step = True
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            m(x).sum().backward()
            opt.step()
        counts.append(lossy_warnings(caught))
        m.zero_grad(set_to_none=True)
    assert counts == [1, 0]
    dense = Two().to(torch.bfloat16).to(device)
    opt = Adam(dense.parameters(), mode="fp32_master")
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        dense(x).sum().backward()
        opt.step()
    assert lossy_warnings(caught) == 0


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("kind", ["adam", "offload"])
def test_load_master_from_pretrained(device, kind, tmp_path):
    torch.manual_seed(0)
    pre = Two().to(torch.bfloat16).to(device)
    want = {n: p.detach().float().cpu() for n, p in pre.named_parameters()}
    single = tmp_path / "model.safetensors"
    save_params(pre, single)
    only_l1 = tmp_path / "partial.safetensors"
    save_params(pre, only_l1, keys={"l1.weight"})
    shard_dir = tmp_path / "sharded"
    shard_dir.mkdir()
    save_params(pre, shard_dir / "model-00001-of-00002.safetensors", keys={"l1.weight"})
    save_params(pre, shard_dir / "model-00002-of-00002.safetensors", keys={"l2.weight"})
    (shard_dir / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": {
        "l1.weight": "model-00001-of-00002.safetensors", "l2.weight": "model-00002-of-00002.safetensors"}}))

    quantize_linears(pre, Int4QWeight, group_size=128)

    def make():
        return Adam(pre.parameters(), mode="fp32_master", lr=1e-3) if kind == "adam" else \
            OffloadAdam(pre, mode="fp32_master", lr=1e-3)

    for source in (single, shard_dir):
        opt = make()
        assert opt.load_master_from_pretrained(source, pre, strict=True) == []
        for name, p in pre.named_parameters():
            st = opt.state[p]
            assert st["master_filled"] is True
            assert torch.equal(st["master_params"].cpu(), want[name])
    opt = make()
    assert opt.load_master_from_pretrained(only_l1, pre) == ["l2.weight"]
    with pytest.raises(ValueError, match="strict=True"):
        opt.load_master_from_pretrained(only_l1, pre, strict=True)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError):
        opt.load_master_from_pretrained(empty, pre)
    # a refilled master silences the warning
    opt = make()
    opt.load_master_from_pretrained(single, pre, strict=True)
    opt.ready_for_optimizer_step = True
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        pre(torch.randn(4, 128, dtype=torch.bfloat16, device=device)).sum().backward()
        opt.step()
    assert lossy_warnings(caught) == 0


def test_load_master_skips_dense_params(tmp_path):
    torch.manual_seed(0)
    m = Block().to(torch.bfloat16)
    save_params(m, tmp_path / "model.safetensors")
    ln = m.ln.weight.data.float().clone()
    quantize_linears(m, Int4QWeight, group_size=128)
    opt = Adam(m.parameters(), mode="fp32_master")
    assert opt.load_master_from_pretrained(tmp_path / "model.safetensors", m) == []
    assert opt.state[m.l1.weight]["master_filled"] is True
    opt._init_state_if_empty(m.ln.weight, opt.state[m.ln.weight])
    assert torch.equal(opt.state[m.ln.weight]["master_params"], ln)
    assert "master_filled" not in opt.state[m.ln.weight]


def test_load_master_state_dict():
    m = build(Int4QWeight, {"group_size": 128}, "cpu", Two)
    for opt in (Adam(m.parameters(), mode="fp32_master"), OffloadAdam(m, mode="fp32_master")):
        with pytest.raises(ValueError, match="strict=True"):
            opt.load_master_state_dict({"l1.weigth": torch.zeros(128, 128)}, m, strict=True)
        (unexpected,) = opt.load_master_state_dict({"l1.weight": torch.full((128, 128), 0.5),
                                                    "ghost.weight": torch.zeros(4)}, m)
        assert unexpected == ["ghost.weight"]
        st = opt.state[m.l1.weight]
        assert st["master_filled"] is True and bool((st["master_params"] == 0.5).all())


@pytest.mark.parametrize("device", DEVICES)
def test_adam_resume_keeps_fp32_master_and_flag(device, tmp_path):
    torch.manual_seed(0)
    pre = Two().to(torch.bfloat16).to(device)
    save_params(pre, tmp_path / "model.safetensors")
    m = build(Int4QWeight, {"group_size": 128}, device, Two)
    opt1 = Adam(m.parameters(), mode="fp32_master", lr=1e-3)
    opt1.load_master_from_pretrained(tmp_path / "model.safetensors", m, strict=True)
    x = torch.randn(4, 128, dtype=torch.bfloat16, device=device)
    m(x).sum().backward()
    opt1.step()
    saved = opt1.state[m.l1.weight]["master_params"].clone()
    sd = opt1.state_dict()
    m2 = build(Int4QWeight, {"group_size": 128}, device, Two)
    opt2 = Adam(m2.parameters(), mode="fp32_master", lr=1e-3)
    opt2.load_state_dict(sd)
    st = opt2.state[m2.l1.weight]
    assert st["master_filled"] is True and st["master_params"].dtype == torch.float32
    assert torch.equal(st["master_params"], saved)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        m2(x).sum().backward()
        opt2.step()
    assert lossy_warnings(caught) == 0
    off = OffloadAdam(m2, mode="fp32_master")
    with pytest.raises(NotImplementedError, match="not supported"):
        off.load_state_dict(off.state_dict())


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cls,kw", FORMATS, ids=IDS)
def test_qat_training_step_requantizes_from_master(device, cls, kw):
    """After a step the packed weight is exactly the quantization of the fp32 master,
    for Adam and for OffloadAdam (whose master lives on the host)."""
    for kind in ("adam", "offload"):
        m = build(cls, kw, device, Block)
        opt = Adam(m.parameters(), mode="fp32_master", lr=1e-2) if kind == "adam" else \
            OffloadAdam(m, mode="fp32_master", lr=1e-2, inplace_param_threshold=0)
        x = torch.randn(8, 256, dtype=torch.bfloat16, device=device)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            for _ in range(2):
                opt.ready_for_optimizer_step = True
                m(x).float().pow(2).mean().backward()
                opt.step()
                m.zero_grad(set_to_none=True)
        if kind == "offload":
            opt.synchronize()
        p = m.l1.weight
        master = opt.state[p]["master_params"].to(device)
        want = cls.from_float(torch.zeros(p.shape, dtype=torch.bfloat16, device=device), **kw)
        want.copy_(master)
        assert torch.equal(p.data.dequantize(), want.dequantize())
        assert opt.state[p]["step"] == 2
