"""The optimizers on HuggingFace modules, which is how the reference is documented to be
used (``AutoModelForCausalLM`` + ``OffloadAdam(model, ...)``): a two-layer
``LlamaForCausalLM`` built from a config (no download) trained for two steps with
``OffloadAdam`` must land on exactly the parameters ``Adam`` of the same mode produces;
a QAT variant with quantized linears must keep packed weights equal to the
re-quantization of the master and export through ``save_quantized_pretrained``."""

import json
import warnings

import pytest
import torch

from offload_adam_b200 import Adam, OffloadAdam
from offload_adam_b200.qweight import Int8QWeight, NVFP4QWeight, quantize_linears, save_quantized_pretrained

transformers = pytest.importorskip("transformers")

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def tiny_hf_llama(device, layers=2):
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=layers,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                   tie_word_embeddings=False, attn_implementation="sdpa", use_cache=False)
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).to(device).train()


def token_batches(n, device):
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 512, (2, 32), generator=g).to(device) for _ in range(n)]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("mode", ["fp32_master", "fp31_master"])
@pytest.mark.parametrize("clip", [None, 1.0])
def test_offload_adam_on_hf_llama_equals_adam(device, mode, clip):
    ga, steps = 2, 2
    data = token_batches(ga * steps, device)
    m_ref, m_off = tiny_hf_llama(device), tiny_hf_llama(device)
    ref = Adam(m_ref.parameters(), lr=1e-3, weight_decay=0.01, mode=mode, decoupled_weight_decay=True)
    off = OffloadAdam(m_off, lr=1e-3, weight_decay=0.01, mode=mode, decoupled_weight_decay=True,
                      max_grad_norm=clip, inplace_param_threshold=1000, chunk_elems=8192)
    for s in range(steps):
        for micro in range(ga):
            off.ready_for_optimizer_step = micro == ga - 1
            (m_off(input_ids=data[s * ga + micro], labels=data[s * ga + micro]).loss / ga).backward()
        off.step()
        # the same gradients for the on-device optimizer: bf16 accumulation over micro-batches
        acc = None
        for micro in range(ga):
            m_ref.zero_grad()
            (m_ref(input_ids=data[s * ga + micro], labels=data[s * ga + micro]).loss / ga).backward()
            gs = [p.grad.detach().clone() for p in m_ref.parameters()]
            acc = gs if acc is None else [(a.float() + g.float()).to(torch.bfloat16) for a, g in zip(acc, gs)]
        if clip is not None:
            total = torch.sqrt(sum((g.float() ** 2).sum() for g in acc))
            coef = torch.clamp(clip / (total + 1e-6), max=1.0)
            # the offloaded optimizer scales in fp32 inside its kernel
            from offload_adam_b200.ops.adam_step import adam_step
            for p, g in zip(m_ref.parameters(), acc):
                st = ref.state[p]
                ref._init_state_if_empty(p, st)
                st["step"] += 1
                tensors = {k: st[k] for k in ref.config["states"]}
                tensors["grad"] = g
                adam_step(mode, p.data, tensors, 1e-3, 0.01, 0.9, 0.999, 1e-8, st["step"],
                          decoupled_weight_decay=True, clip_coef=coef.reshape(1))
        else:
            for p, g in zip(m_ref.parameters(), acc):
                p.grad = g
            ref.step()
    off.synchronize()
    names = [n for n, _ in m_ref.named_parameters()]
    for name, p, q in zip(names, m_ref.parameters(), m_off.parameters()):
        if clip is None:
            assert torch.equal(p, q), name
        else:  # the squared norm is summed in another order: same up to the last bits of the coefficient
            assert torch.allclose(p.float(), q.float(), atol=1e-5, rtol=0), name


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cls", [NVFP4QWeight, Int8QWeight], ids=["nvfp4", "int8"])
def test_qat_on_hf_llama_and_export(device, cls, tmp_path):
    model = tiny_hf_llama(device)
    report = quantize_linears(model, cls, skip_patterns=("lm_head",), update_hf_config=True)
    assert len(report.quantized) == 2 * 7 and report.excluded == ["lm_head"]
    opt = OffloadAdam(model, lr=1e-3, mode="fp32_master", inplace_param_threshold=1000, chunk_elems=8192)
    data = token_batches(2, device)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for b in data:
            opt.ready_for_optimizer_step = True
            model(input_ids=b, labels=b).loss.backward()
            opt.step()
    opt.synchronize()
    p = model.model.layers[0].mlp.up_proj.weight
    want = cls.from_float(torch.zeros(p.shape, dtype=torch.bfloat16, device=device))
    want.copy_(opt.state[p]["master_params"].to(device))
    assert torch.equal(p.data.dequantize(), want.dequantize())
    save_quantized_pretrained(model, tmp_path / "export", cls, skip_patterns=("lm_head",))
    cfg = json.loads((tmp_path / "export" / "config.json").read_text())
    assert cfg["quantization_config"]["quant_method"] == "compressed-tensors"
    from safetensors import safe_open
    files = list((tmp_path / "export").glob("*.safetensors"))
    assert files
    with safe_open(str(files[0]), "pt") as f:
        keys = set(f.keys())
    assert "model.layers.0.mlp.up_proj.weight_packed" in keys and "model.layers.0.mlp.up_proj.weight" not in keys


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("tied", [False, True])
def test_chunked_loss_of_hf_model_equals_its_own_loss(device, tied):
    """``causal_lm_loss`` (decoder as usual, head and loss chunk by chunk) against the
    module's own full-logits loss: same value, same gradients, also with tied embeddings
    and ignored labels."""
    from offload_adam_b200.models.hf import causal_lm_loss, supports_chunked_loss
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                   tie_word_embeddings=tied, attn_implementation="sdpa", use_cache=False)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).to(torch.float32).to(device).train()
    assert supports_chunked_loss(model)
    ids = token_batches(1, device)[0]
    labels = ids.clone()
    labels[0, 5:9] = -100
    want = model(input_ids=ids, labels=labels).loss
    want.backward()
    g_want = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad(set_to_none=True)
    got = causal_lm_loss(model, ids, labels, chunk=24)   # 64 rows: two full chunks and a tail
    got.backward()
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    for n, p in model.named_parameters():
        torch.testing.assert_close(p.grad, g_want[n], rtol=2e-4, atol=1e-6, msg=n)
    # a head this function cannot take apart falls back to the module's own loss
    model.lm_head.bias = torch.nn.Parameter(torch.zeros(512, device=device))
    assert not supports_chunked_loss(model)
    torch.testing.assert_close(causal_lm_loss(model, ids, labels), model(input_ids=ids, labels=labels).loss)
