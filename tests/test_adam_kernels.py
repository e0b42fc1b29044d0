"""Numerics of the fused Adam step: CPU oracle properties and, on a GPU, the
sm_100a kernels against the fp32 PyTorch restatement (bit for bit)."""

import numpy as np
import pytest
import torch

from offload_adam_b200.ops import oracle
from offload_adam_b200.ops.adam_step import STEP_FNS, adam_step
from offload_adam_b200.ops.oracle import MODE_IDS, beta_hat

MODES = list(MODE_IDS)


def make_states(n, mode, device="cpu", seed=0, warm=True):
    g = torch.Generator().manual_seed(seed)
    p = (torch.randn(n, generator=g) * 0.05).to(torch.bfloat16)
    st = {
        "grad": (torch.randn(n, generator=g) * 1e-2).to(torch.bfloat16),
        "exp_avg": (torch.randn(n, generator=g) * 1e-3).to(torch.bfloat16) if warm else torch.zeros(n, dtype=torch.bfloat16),
        "exp_avg_sq": (torch.rand(n, generator=g) * 1e-5).to(torch.bfloat16) if warm else torch.zeros(n, dtype=torch.bfloat16),
    }
    if mode == "fp32_master":
        st["master_params"] = p.float() + torch.randn(n, generator=g) * 1e-5
    elif mode in ("fp31_master", "fp32_master_custom_rounding"):
        st["rounding_error"] = torch.randint(-3000, 3000, (n,), generator=g, dtype=torch.int16)
    return p.to(device), {k: v.to(device) for k, v in st.items()}


def clone_states(p, st):
    return p.clone(), {k: v.clone() for k, v in st.items()}


# ------------------------------------------------------------------ CPU oracle
def test_philox_known_answer():
    x, y, z, w = oracle.philox4x32_10(np.array([0], dtype=np.uint64), 0)
    assert [int(x[0]), int(y[0]), int(z[0]), int(w[0])] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def test_beta_hat_first_step_is_plain_copy():
    assert beta_hat(0.9, 1) == 0.0
    p, st = make_states(64, "fp32_master", warm=False)
    g = st["grad"].float()
    adam_step("fp32_master", p, st, 1e-3, 0.0, 0.9, 0.999, 1e-8, 1)
    assert torch.equal(st["exp_avg"], g.to(torch.bfloat16))
    assert torch.equal(st["exp_avg_sq"], (g * g).to(torch.bfloat16))


def test_fp32_master_tracks_torch_adamw():
    torch.manual_seed(0)
    w = torch.randn(257) * 0.1
    ref = w.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    p = w.to(torch.bfloat16)
    st = {"exp_avg": torch.zeros(257, dtype=torch.bfloat16), "exp_avg_sq": torch.zeros(257, dtype=torch.bfloat16),
          "master_params": w.clone()}
    for step in range(1, 21):
        g = torch.randn(257) * 0.01
        gb = g.to(torch.bfloat16)
        ref.grad = gb.float()
        opt.step()
        st["grad"] = gb
        adam_step("fp32_master", p, st, 1e-2, 0.1, 0.9, 0.99, 1e-8, step, decoupled_weight_decay=True)
    # moments are stored in bf16, so agreement is at the bf16-moment level
    assert torch.allclose(st["master_params"], ref.detach(), rtol=0, atol=2e-3)
    assert torch.equal(p, st["master_params"].to(torch.bfloat16))


@pytest.mark.parametrize("fn", ["fp31", "custom"])
def test_decompose_reconstruct(fn):
    torch.manual_seed(1)
    x = torch.cat([torch.randn(4096) * 10 ** torch.randint(-6, 3, (4096,)).float(),
                   torch.tensor([0.0, -0.0, 1.0, -1.0, 3.0e-39])])
    if fn == "fp31":
        q, e = oracle.fp31_decompose(x)
        back = oracle.fp31_reconstruct(q, e)
        assert torch.equal(back, oracle.round_to_fp31(x))
        # at most the last bit of the fp32 mantissa is lost
        assert (back.view(torch.int32) - x.view(torch.int32)).abs().max() <= 1
    else:
        q, e = oracle.custom_decompose(x)
        back = oracle.custom_reconstruct(q, e)
        assert torch.equal(back.view(torch.int32), x.view(torch.int32))
    assert q.dtype == torch.bfloat16 and e.dtype == torch.int16


def test_stochastic_rounding_unbiased_and_seeded():
    x = torch.full((200000,), 1.0 + 2.0**-10)  # sits 1/8 of the way between two bf16 values
    r1 = oracle.bf16_sr(x, oracle.sr_random_words(x.numel(), seed=7))
    r2 = oracle.bf16_sr(x, oracle.sr_random_words(x.numel(), seed=7))
    r3 = oracle.bf16_sr(x, oracle.sr_random_words(x.numel(), seed=8))
    assert torch.equal(r1, r2) and not torch.equal(r1, r3)
    assert set(r1.float().unique().tolist()) == {1.0, 1.0078125}
    assert abs(r1.float().mean().item() - x[0].item()) < 2e-5
    # chunking must not change the stream
    a = oracle.sr_random_words(100, seed=3, elem_offset=0)
    b = oracle.sr_random_words(60, seed=3, elem_offset=40)
    assert torch.equal(a[40:], b)


def test_public_step_functions_signature():
    for mode, fn in STEP_FNS.items():
        p, st = make_states(40, mode)
        before = p.clone()
        fn(p, st, 1e-2, 0.01, 0.9, 0.999, 1e-8, 3, decoupled_weight_decay=True)
        assert not torch.equal(p, before)


# ------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("decoupled", [False, True])
@pytest.mark.parametrize("n", [1, 7, 8, 1000, 4099, 1 << 20])
def test_kernel_matches_oracle_bitwise(mode, decoupled, n):
    p, st = make_states(n, mode, seed=n)
    pc, stc = clone_states(p, st)
    pg, stg = p.cuda(), {k: v.cuda() for k, v in st.items()}
    kw = dict(decoupled_weight_decay=decoupled, seed=1234)
    adam_step(mode, pc, stc, 3e-3, 0.05, 0.9, 0.95, 1e-8, 5, **kw)
    adam_step(mode, pg, stg, 3e-3, 0.05, 0.9, 0.95, 1e-8, 5, **kw)
    torch.cuda.synchronize()
    assert torch.equal(pg.cpu().view(torch.int16), pc.view(torch.int16))
    for k in stc:
        if k == "grad":
            continue
        a, b = stg[k].cpu(), stc[k]
        if a.dtype in (torch.bfloat16,):
            a, b = a.view(torch.int16), b.view(torch.int16)
        elif a.dtype == torch.float32:
            a, b = a.view(torch.int32), b.view(torch.int32)
        assert torch.equal(a, b), k


@pytest.mark.gpu
@pytest.mark.parametrize("mode", MODES)
def test_kernel_clip_second_grad_offset_and_unaligned(mode):
    n = 5003
    p, st = make_states(n + 3, mode, seed=3)
    g2 = (torch.randn(n + 3) * 1e-2).to(torch.bfloat16)
    clip = torch.tensor([0.37])
    # unaligned views (offset by 3 elements) force the scalar path on the GPU
    sl = slice(3, None)
    pc, stc = p.clone()[sl], {k: v.clone()[sl] for k, v in st.items()}
    pg_full, stg_full = p.cuda(), {k: v.cuda() for k, v in st.items()}
    pg, stg = pg_full[sl], {k: v[sl] for k, v in stg_full.items()}
    kw = dict(decoupled_weight_decay=True, seed=99, elem_offset=40)
    adam_step(mode, pc, stc, 1e-3, 0.01, 0.9, 0.999, 1e-8, 2, clip_coef=clip, grad2=g2[sl].clone(), **kw)
    adam_step(mode, pg, stg, 1e-3, 0.01, 0.9, 0.999, 1e-8, 2, clip_coef=clip.cuda(), grad2=g2.cuda()[sl], **kw)
    torch.cuda.synchronize()
    assert torch.equal(pg.cpu().view(torch.int16), pc.view(torch.int16))
    assert torch.equal(stg["exp_avg"].cpu().view(torch.int16), stc["exp_avg"].view(torch.int16))
    assert torch.equal(stg["exp_avg_sq"].cpu().view(torch.int16), stc["exp_avg_sq"].view(torch.int16))


@pytest.mark.gpu
def test_sr_stream_independent_of_chunking():
    n = 1 << 16
    p, st = make_states(n, "stochastic_rounding", seed=5)
    p1, st1 = p.cuda(), {k: v.cuda() for k, v in st.items()}
    p2, st2 = p.cuda(), {k: v.cuda() for k, v in st.items()}
    adam_step("stochastic_rounding", p1, st1, 1e-3, 0.0, 0.9, 0.999, 1e-8, 2, seed=11)
    h = n // 2
    for lo in (0, h):
        adam_step("stochastic_rounding", p2[lo:lo + h], {k: v[lo:lo + h] for k, v in st2.items()},
                  1e-3, 0.0, 0.9, 0.999, 1e-8, 2, seed=11, elem_offset=lo)
    torch.cuda.synchronize()
    assert torch.equal(p1, p2)


@pytest.mark.gpu
def test_amax_side_output():
    n = 10000
    p, st = make_states(n, "fp32_master", seed=8)
    pg, stg = p.cuda(), {k: v.cuda() for k, v in st.items()}
    amax = torch.zeros(1, device="cuda")
    adam_step("fp32_master", pg, stg, 1e-3, 0.0, 0.9, 0.999, 1e-8, 2, amax=amax)
    torch.cuda.synchronize()
    assert amax.item() == stg["master_params"].abs().max().item()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", MODES)
def test_multi_tensor_matches_single(mode):
    from offload_adam_b200.ops.grad_ops import MultiTensorAdam
    sizes = [1, 5, 64, 4096, 9000, 12345]
    singles, entries = [], []
    for i, n in enumerate(sizes):
        p, st = make_states(n, mode, seed=20 + i)
        singles.append((p.cuda(), {k: v.cuda() for k, v in st.items()}))
        pg, stg = p.cuda(), {k: v.cuda() for k, v in st.items()}
        extra = stg.get("master_params", stg.get("rounding_error"))
        entries.append({"param": pg, "grad": stg["grad"], "exp_avg": stg["exp_avg"],
                        "exp_avg_sq": stg["exp_avg_sq"], "extra": extra})
    clip = torch.tensor([0.5], device="cuda")
    mt = MultiTensorAdam(entries, mode)
    mt.step(2e-3, 0.01, 0.9, 0.999, 1e-8, 4, True, clip_coef=clip, seed=77, zero_grad=True)
    off = 0
    for (p, st), e, n in zip(singles, entries, sizes):
        adam_step(mode, p, st, 2e-3, 0.01, 0.9, 0.999, 1e-8, 4, decoupled_weight_decay=True,
                  clip_coef=clip, seed=77, elem_offset=off)
        off += (n + 7) // 8 * 8
        assert torch.equal(p, e["param"])
        assert torch.equal(st["exp_avg"], e["exp_avg"]) and torch.equal(st["exp_avg_sq"], e["exp_avg_sq"])
        assert e["grad"].abs().sum().item() == 0
