"""Loss of a HuggingFace causal LM without materialising its logits.

``model(input_ids=ids, labels=ids).loss`` of a stock HuggingFace module builds the full
``(tokens, vocab)`` logits in fp32 and their gradient: 2 x 2.1 GB for 4096 tokens of a
128k vocabulary, live across the whole backward pass of the decoder stack.  The
reference's example trainer offers Liger's fused linear cross-entropy for this, wired
for Qwen3 only (reference: examples/e2e_train/train.py:76-115).  ``causal_lm_loss`` does
the same for any HF causal LM that exposes its decoder as ``.model`` and an unbiased
``nn.Linear`` ``.lm_head`` (Llama, Qwen2/3, Mistral, Gemma, ...): the decoder runs as
usual, the head and the loss run chunk by chunk through
:func:`offload_adam_b200.models.llama.chunked_linear_cross_entropy`, which forms the
gradients of the hidden states and of the head weight in the same pass.  Tied
embeddings work unchanged (the head weight is the embedding parameter; autograd adds
both contributions)."""

from __future__ import annotations

import torch

from .llama import chunked_linear_cross_entropy


def supports_chunked_loss(hf_model) -> bool:
    """True when ``causal_lm_loss`` can bypass the module's own head and loss."""
    head = getattr(hf_model, "lm_head", None)
    body = getattr(hf_model, "model", None)
    if body is None or not isinstance(head, torch.nn.Linear) or head.bias is not None:
        return False
    # a quantized head (tensor subclass) keeps its own matmul path
    if type(head.weight.data) is not torch.Tensor:
        return False
    # heads followed by a soft cap or a scale (Gemma-2, Cohere) are not a plain linear + CE
    cfg = getattr(hf_model, "config", None)
    if getattr(cfg, "final_logit_softcapping", None) or getattr(cfg, "logit_scale", None):
        return False
    return True


def causal_lm_loss(hf_model, input_ids, labels=None, chunk: int = 2048, **model_kwargs):
    """Mean next-token cross-entropy of ``hf_model`` on ``input_ids`` (labels shifted here,
    ``-100`` ignored, as in HuggingFace's own loss).  Falls back to the module's own loss
    when the model does not have the plain ``.model`` / ``.lm_head`` structure."""
    labels = input_ids if labels is None else labels
    if not supports_chunked_loss(hf_model):
        return hf_model(input_ids=input_ids, labels=labels, **model_kwargs).loss
    h = hf_model.model(input_ids=input_ids, **model_kwargs).last_hidden_state
    B, S, H = h.shape
    shift = torch.full_like(labels, -100)
    shift[:, :-1] = labels[:, 1:]
    return chunked_linear_cross_entropy(h.reshape(B * S, H), hf_model.lm_head.weight, shift.reshape(-1), chunk)
