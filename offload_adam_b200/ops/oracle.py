"""Plain PyTorch fp32 restatement of every optimizer kernel.

Two jobs: (1) the numerics oracle that the CUDA kernels are tested against, op
by op in fp32 with the same rounding points, so that the deterministic modes
compare bit for bit; (2) the implementation used for CPU tensors (unit tests
and multi-process gloo tests run the full optimizers on CPU through it).

Formulas: reference src/offload_adam/kernels/stochastic_rounding.py:25-79,
fp32_master.py:40-59, fp31_master.py:26-54, fp32_master_custom_rounding.py:33-54.
"""

from __future__ import annotations

import numpy as np
import torch

MODE_IDS = {
    "stochastic_rounding": 0,
    "fp32_master": 1,
    "fp31_master": 2,
    "fp32_master_custom_rounding": 3,
}
MODE_NAMES = {v: k for k, v in MODE_IDS.items()}


def beta_hat(beta: float, step: int) -> float:
    """EMA coefficient with the bias correction folded in (host double math).

    (reference: kernels/fp32_master.py:74-75).  At step 1 it is 0, so m = g and
    v = g*g; the stored moments are already bias-corrected.
    """
    bs = beta**step
    return (bs - beta) / (bs - 1)


# ----------------------------------------------------------------------------
# Philox4x32-10 (counter = (lo, hi, 0, 0), key = seed split in two words)
# ----------------------------------------------------------------------------
_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter: np.ndarray, seed: int):
    counter = counter.astype(np.uint64)
    c0 = counter & _MASK32
    c1 = (counter >> np.uint64(32)) & _MASK32
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    seed &= (1 << 64) - 1
    k0 = seed & 0xFFFFFFFF
    k1 = (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def sr_random_words(n: int, seed: int, elem_offset: int = 0) -> torch.Tensor:
    """16-bit random word of each of n consecutive elements (int32 tensor, CPU)."""
    G = np.arange(elem_offset, elem_offset + n, dtype=np.uint64)
    ctr = G >> np.uint64(3)
    # one Philox call per group of 8 elements
    uniq, inv = np.unique(ctr, return_inverse=True)
    words = philox4x32_10(uniq, seed)
    W = np.stack(words, axis=0)  # (4, groups)
    j = (G & np.uint64(7)).astype(np.int64)
    w = W[j >> 1, inv]
    r = (w >> ((j & 1) * 16).astype(np.uint64)) & np.uint64(0xFFFF)
    return torch.from_numpy(r.astype(np.int32))


# ----------------------------------------------------------------------------
# bit helpers (operate on int32 views of fp32 tensors)
# ----------------------------------------------------------------------------
def _bits(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.int32)


def _from_bits(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float32)


def bf16_sr(x: torch.Tensor, rand16: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16: truncate, then one step away from zero iff rand16 < low 16 bits."""
    b = _bits(x)
    frac = b & 0xFFFF
    trunc = b & -0x10000
    up = rand16.to(b.device) < frac
    r = torch.where(up, trunc + 0x10000, trunc)
    return _from_bits(r).to(torch.bfloat16)


def round_to_fp31(x: torch.Tensor) -> torch.Tensor:
    b = _bits(x)
    up = (b & 1) & ((b >> 1) & 1)
    return _from_bits(((b >> 1) + up) << 1)


def fp31_decompose(x: torch.Tensor):
    x31 = round_to_fp31(x)
    q = x31.to(torch.bfloat16)
    err = (_bits(x31) - _bits(q.float())) >> 1
    return q, err.to(torch.int16)


def fp31_reconstruct(q: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
    return _from_bits(_bits(q.float()) + (err.to(torch.int32) << 1))


def custom_decompose(x: torch.Tensor):
    b = _bits(x)
    hi = (b + 0x8000) >> 16  # arithmetic shift keeps the sign bits
    qbits = hi << 16
    q = _from_bits(qbits).to(torch.bfloat16)  # exact: low 16 bits are zero
    err = (b - qbits).to(torch.int16)
    return q, err


def custom_reconstruct(q: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
    return _from_bits(_bits(q.float()) + err.to(torch.int32))


# ----------------------------------------------------------------------------
# Adam step
# ----------------------------------------------------------------------------
def _f32(x, device):
    return torch.tensor(float(x), dtype=torch.float32, device=device)


def _sqrt_rn(x: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 square root.  PyTorch's vectorised CPU sqrt is not
    always correctly rounded; numpy's is, and so is the CUDA one."""
    if x.device.type == "cpu":
        return torch.from_numpy(np.asarray(np.sqrt(x.contiguous().numpy()), dtype=np.float32)).reshape(x.shape)
    return torch.sqrt(x)


@torch.no_grad()
def adam_step(
    mode,
    p,
    g,
    m,
    v,
    extra,
    lr,
    wd,
    beta1_hat,
    beta2_hat,
    eps,
    decoupled,
    clip=None,
    g2=None,
    seed=0,
    elem_offset=0,
    amax=None,
):
    """In-place step on flat or shaped tensors; same contract as ``_C.adam_step``."""
    if isinstance(mode, str):
        mode = MODE_IDS[mode]
    dev = g.device
    gf = g.detach().reshape(-1).float()
    if g2 is not None:
        gf = (gf + g2.detach().reshape(-1).to(dev).float()).to(torch.bfloat16).float()
    if clip is not None:
        gf = gf * clip.detach().to(dev).float().reshape(())
    mf = m.reshape(-1).float()
    vf = v.reshape(-1).float()
    if mode == 0:
        pf = p.detach().reshape(-1).float()
    elif mode == 1:
        pf = extra.reshape(-1).clone()
    elif mode == 2:
        pf = fp31_reconstruct(p.detach().reshape(-1), extra.reshape(-1))
    else:
        pf = custom_reconstruct(p.detach().reshape(-1), extra.reshape(-1))

    lr32, wd32, eps32 = _f32(lr, dev), _f32(wd, dev), _f32(eps, dev)
    c1 = _f32(1.0, dev) - _f32(beta1_hat, dev)
    c2 = _f32(1.0, dev) - _f32(beta2_hat, dev)
    if decoupled:
        pf = pf - (lr32 * wd32) * pf
    else:
        gf = gf + wd32 * pf
    mf = mf + c1 * (gf - mf)
    vf = vf + c2 * (gf * gf - vf)
    denom = _sqrt_rn(vf) + eps32
    pf = pf - (lr32 * mf) / denom

    m.reshape(-1).copy_(mf.to(torch.bfloat16))
    v.reshape(-1).copy_(vf.to(torch.bfloat16))
    if amax is not None:
        amax.copy_(torch.maximum(amax.reshape(()), pf.abs().max().to(amax.device)).reshape(amax.shape))
    if mode == 0:
        rnd = sr_random_words(pf.numel(), seed, elem_offset)
        p.detach().reshape(-1).copy_(bf16_sr(pf, rnd))
    elif mode == 1:
        extra.reshape(-1).copy_(pf)
        if p is not None:
            p.detach().reshape(-1).copy_(pf.to(torch.bfloat16))
    elif mode == 2:
        q, err = fp31_decompose(pf)
        p.detach().reshape(-1).copy_(q)
        extra.reshape(-1).copy_(err)
    else:
        q, err = custom_decompose(pf)
        p.detach().reshape(-1).copy_(q)
        extra.reshape(-1).copy_(err)


@torch.no_grad()
def grad_accumulate(out, a, b=None, want_sumsq=False):
    """out = bf16(a + b) (b None: out = a); returns sum of squares of the result (fp32)."""
    r = a.detach().reshape(-1)
    if b is not None:
        r = (r.float() + b.detach().reshape(-1).to(r.device).float()).to(torch.bfloat16)
    if out is not None:
        out.reshape(-1).copy_(r)
    if want_sumsq:
        return (r.float() * r.float()).sum(dtype=torch.float32)
    return None


def clip_coef_from_sq(total_sq: torch.Tensor, max_norm: float):
    """(reference: offload_adam.py:560-561) clamp(max / (norm + 1e-6), max=1)."""
    norm = _sqrt_rn(total_sq.float())
    coef = torch.clamp(_f32(max_norm, norm.device) / (norm + _f32(1e-6, norm.device)), max=1.0)
    return coef, norm
