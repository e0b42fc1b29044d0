"""The allocation-free squared-norm entry point, called the way a host without PyTorch
bindings would call it: through its exported C symbol.  Its result is compared with
the scratch-tensor entry point the optimizers use, on two calls in a row (the second
call finds the built-in scratch array as the first one left it)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 65536 * 8192


def load_symbol():
    from offload_adam_b200 import _ext
    mod = _ext.load(required=True)
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.oab_sumsq_bf16_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_char_p, ctypes.c_int]
    return fn


def call(fn, x, n, out, stream=None):
    err = ctypes.create_string_buffer(256)
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    rc = fn(x.data_ptr() if x is not None else None, n, out.data_ptr(), handle, err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("n", [1, 17, 8192, 8193, 1_000_003, 40_000_000])
def test_matches_scratch_tensor_entry_point_twice(n):
    from offload_adam_b200.ops import grad_ops
    fn = load_symbol()
    torch.manual_seed(n)
    x = (torch.randn(n, device="cuda") * 0.05).to(torch.bfloat16)
    want = torch.zeros(1, device="cuda")
    grad_ops.grad_accumulate(None, x, None, sumsq=want, scratch=grad_ops.sumsq_scratch("cuda"))
    exact = (x.double() ** 2).sum().item()
    results = []
    for _ in range(2):
        out = torch.full((1,), -1.0, device="cuda")
        rc, msg = call(fn, x, n, out)
        assert rc == 0, msg
        torch.cuda.synchronize()
        results.append(out.item())
    tol = 2e-6 * exact + 1e-12
    assert abs(results[0] - want.item()) <= tol
    assert abs(results[0] - exact) <= tol
    assert results[0] == results[1]  # same order of additions on both calls


def test_unaligned_input_side_stream_and_empty():
    fn = load_symbol()
    base = (torch.randn(50_001, device="cuda") * 0.1).to(torch.bfloat16)
    x = base[1:]  # 2-byte aligned only: scalar path
    out = torch.zeros(1, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    rc, msg = call(fn, x, x.numel(), out, stream=side)
    assert rc == 0, msg
    side.synchronize()
    exact = (x.double() ** 2).sum().item()
    assert abs(out.item() - exact) <= 2e-6 * exact
    out.fill_(5.0)
    rc, msg = call(fn, None, 0, out)
    torch.cuda.synchronize()
    assert rc == 0 and out.item() == 0.0


def test_rejects_oversize_and_bad_arguments_without_launching():
    fn = load_symbol()
    x = torch.ones(16, dtype=torch.bfloat16, device="cuda")
    out = torch.full((1,), 7.0, device="cuda")
    rc, msg = call(fn, x, MAX_ELEMS + 1, out)
    assert rc == 2 and "exceeds" in msg and str(MAX_ELEMS) in msg
    rc, msg = call(fn, x, -1, out)
    assert rc == 1 and "negative" in msg
    err = ctypes.create_string_buffer(64)
    assert fn(x.data_ptr(), 16, None, None, err, 64) == 1
    torch.cuda.synchronize()
    assert out.item() == 7.0  # nothing ran
    rc, msg = call(fn, x, 16, out)
    torch.cuda.synchronize()
    assert rc == 0 and out.item() == 16.0
