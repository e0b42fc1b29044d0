"""Self-contained Llama-style causal LM used by the examples and benchmarks.

The reference's examples train a HuggingFace ``AutoModelForCausalLM`` with SDPA
attention, gradient checkpointing and a fused linear cross-entropy
(reference: examples/e2e_train/train.py:106-129).  This module provides the same
ingredients without external model code: RMSNorm, rotary embeddings, grouped
query attention through ``scaled_dot_product_attention``, SwiGLU, optional
per-layer activation checkpointing and a chunked linear + cross-entropy head
that never materialises the full ``(tokens, vocab)`` logits.

Parameter names and shapes match the HF Llama layout (``model.embed_tokens``,
``model.layers.N.self_attn.{q,k,v,o}_proj``, ``mlp.{gate,up,down}_proj``,
``input_layernorm``, ``post_attention_layernorm``, ``model.norm``, ``lm_head``)
so checkpoints and the quantization name filters line up.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    tie_embeddings: bool = False
    init_std: float = 0.02
    ce_chunk: int = 2048  # rows of the logits computed at a time by the loss head
    head_dim_override: Optional[int] = None  # Qwen3: 128 whatever hidden_size / num_heads is
    qk_norm: bool = False  # Qwen3: RMSNorm over head_dim on queries and keys before RoPE

    @property
    def head_dim(self):
        return self.head_dim_override or self.hidden_size // self.num_heads


def llama3_8b(**kw) -> LlamaConfig:
    return LlamaConfig(**kw)


def llama3_70b(**kw) -> LlamaConfig:
    base = dict(hidden_size=8192, intermediate_size=28672, num_layers=80, num_heads=64, num_kv_heads=8)
    base.update(kw)
    return LlamaConfig(**base)


def qwen3_8b(**kw) -> LlamaConfig:
    """Qwen3-8B shape, the model of the reference's published tables (reference:
    examples/e2e_train/README.md:36-54): 36 layers, hidden 4096, 32 query / 8 KV heads
    of 128, SwiGLU 12288, vocabulary 151936, RoPE theta 1e6, RMSNorm on q and k."""
    base = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_layers=36, num_heads=32,
                num_kv_heads=8, rope_theta=1e6, rms_eps=1e-6, head_dim_override=128, qk_norm=True)
    base.update(kw)
    return LlamaConfig(**base)


def tiny_llama(**kw) -> LlamaConfig:
    """2 layers, hidden 256, 4 heads, SwiGLU 688, vocab 1024, tied embeddings."""
    base = dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_layers=2, num_heads=4,
                num_kv_heads=4, rope_theta=1e4, tie_embeddings=True, ce_chunk=128)
    base.update(kw)
    return LlamaConfig(**base)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def _rope_tables(seq_len, head_dim, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    ang = torch.outer(t, inv)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def _apply_rope(x, cos, sin):
    # x: (B, H, S, D); rotate-half convention
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return x * cos + rot * sin


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        h, d = cfg.hidden_size, cfg.head_dim
        self.nh, self.nkv, self.hd = cfg.num_heads, cfg.num_kv_heads, d
        self.q_proj = nn.Linear(h, self.nh * d, bias=False)
        self.k_proj = nn.Linear(h, self.nkv * d, bias=False)
        self.v_proj = nn.Linear(h, self.nkv * d, bias=False)
        self.o_proj = nn.Linear(self.nh * d, h, bias=False)
        if cfg.qk_norm:  # parameter names as in HF Qwen3: self_attn.q_norm / k_norm
            self.q_norm = RMSNorm(d, cfg.rms_eps)
            self.k_norm = RMSNorm(d, cfg.rms_eps)
        else:
            self.q_norm = self.k_norm = None

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        q = self.q_proj(x).view(B, S, self.nh, self.hd)
        k = self.k_proj(x).view(B, S, self.nkv, self.hd)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        v = self.v_proj(x).view(B, S, self.nkv, self.hd).transpose(1, 2)
        q = _apply_rope(q, cos, sin)
        k = _apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.nh != self.nkv)
        return self.o_proj(o.transpose(1, 2).reshape(B, S, self.nh * self.hd))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class DecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.mlp = MLP(cfg)

    def forward(self, x, cos, sin):
        x = x + self.self_attn(self.input_layernorm(x), cos, sin)
        return x + self.mlp(self.post_attention_layernorm(x))


class _ChunkedLinearCE(torch.autograd.Function):
    """mean cross-entropy of ``h @ W^T`` against ``labels`` (ignore_index=-100),
    computed chunk by chunk.  Gradients with respect to ``h`` and ``W`` are formed
    in the same pass and only scaled in backward, so the logits of a chunk are
    live for one chunk only."""

    @staticmethod
    def forward(ctx, h, weight, labels, chunk):
        N, H = h.shape
        valid = labels != -100
        n_valid = valid.sum().clamp(min=1)
        loss = torch.zeros((), dtype=torch.float32, device=h.device)
        gh = torch.empty_like(h)
        gw = torch.zeros(weight.shape, dtype=torch.float32, device=h.device)
        inv = 1.0 / n_valid.float()
        for s in range(0, N, chunk):
            e = min(N, s + chunk)
            logits = (h[s:e] @ weight.T).float()
            lab = labels[s:e]
            lse = torch.logsumexp(logits, dim=-1)
            msk = valid[s:e]
            safe = lab.clamp(min=0)
            picked = logits.gather(1, safe[:, None]).squeeze(1)
            loss += ((lse - picked) * msk).sum()
            probs = torch.softmax(logits, dim=-1)
            probs.scatter_add_(1, safe[:, None], -torch.ones_like(picked)[:, None])
            probs *= (msk.float() * inv)[:, None]
            d = probs.to(h.dtype)
            gh[s:e] = d @ weight
            gw.add_(d.T @ h[s:e])
        ctx.save_for_backward(gh, gw.to(weight.dtype))
        return loss * inv

    @staticmethod
    def backward(ctx, g):
        gh, gw = ctx.saved_tensors
        return gh * g.to(gh.dtype), gw * g.to(gw.dtype), None, None


def chunked_linear_cross_entropy(h, weight, labels, chunk=2048):
    return _ChunkedLinearCE.apply(h, weight, labels, chunk)


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(cfg) for _ in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)


class LlamaForCausalLM(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.config = cfg
        self.model = LlamaModel(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.gradient_checkpointing = False
        self._rope = None
        self.reset_parameters()

    def reset_parameters(self):
        std = self.config.init_std
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=std)

    def gradient_checkpointing_enable(self):
        self.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False

    def _rope_for(self, S, device, dtype):
        key = (S, device, dtype)
        if self._rope is None or self._rope[0] != key:
            cos, sin = _rope_tables(S, self.config.head_dim, self.config.rope_theta, device)
            self._rope = (key, cos.to(dtype), sin.to(dtype))
        return self._rope[1], self._rope[2]

    def hidden_states(self, input_ids):
        x = self.model.embed_tokens(input_ids)
        cos, sin = self._rope_for(input_ids.shape[1], x.device, x.dtype)
        for layer in self.model.layers:
            if self.gradient_checkpointing and self.training:
                x = checkpoint(layer, x, cos, sin, use_reentrant=False)
            else:
                x = layer(x, cos, sin)
        return self.model.norm(x)

    def forward(self, input_ids, labels: Optional[torch.Tensor] = None):
        """Returns the mean next-token loss when ``labels`` is given (labels are
        shifted here, as in HF models), else the full logits."""
        h = self.hidden_states(input_ids)
        if labels is None:
            return self.lm_head(h)
        B, S, H = h.shape
        shift = torch.full_like(labels, -100)
        shift[:, :-1] = labels[:, 1:]
        return chunked_linear_cross_entropy(h.reshape(B * S, H), self.lm_head.weight,
                                            shift.reshape(-1), self.config.ce_chunk)


def build_llama(cfg: LlamaConfig, device="cuda", dtype=torch.bfloat16, seed=0, symmetric_group=None,
                symmetric_threshold=1024 * 1024) -> LlamaForCausalLM:
    """Random-init model (N(0, init_std), norms at 1) created directly on ``device`` and
    directly in ``dtype``: no fp32 copy of the weights ever exists (a 70B model would not
    fit otherwise).  With ``symmetric_group`` (a process group) the large parameters are
    created in symmetric memory, where the peer-memory path of ``DistributedOffloadAdam``
    wants them, so that no second copy of the weights is needed when the optimizer is
    built (``parallel.symm.materialize_in_symmetric_memory``)."""
    gen_state = torch.random.get_rng_state()
    default_dtype = torch.get_default_dtype()
    torch.manual_seed(seed)
    try:
        torch.set_default_dtype(dtype)
        if symmetric_group is None:
            with torch.device(device):
                model = LlamaForCausalLM(cfg)
            model = model.to(dtype)
        else:
            from ..parallel.symm import materialize_in_symmetric_memory
            with torch.device("meta"):
                model = LlamaForCausalLM(cfg)
            materialize_in_symmetric_memory(model, device, symmetric_group, symmetric_threshold, dtype)
            with torch.no_grad():
                for p in model.parameters():
                    if p.dim() == 1:
                        p.fill_(1.0)  # norm weights
                model.reset_parameters()
    finally:
        torch.set_default_dtype(default_dtype)
        torch.random.set_rng_state(gen_state)
    return model
