"""Kernel micro-benchmarks with roofline fractions.

    python -m offload_adam_b200.utils.microbench adam_step --mode fp32_master --elems 268435456
    python -m offload_adam_b200.utils.microbench staged_step --mode fp32_master --elems 134217728
    python -m offload_adam_b200.utils.microbench accumulate --elems 268435456
    python -m offload_adam_b200.utils.microbench quant --format nvfp4 --rows 14336 --cols 4096
    python -m offload_adam_b200.utils.microbench quant --format nvfp4 --impl reference   # the reference's Triton kernels
    python -m offload_adam_b200.utils.microbench quant_table        # every format x shape x input dtype x implementation
    python -m offload_adam_b200.utils.microbench adam_quant --format int4 --world 8      # fused step + re-quantize + push
    python -m offload_adam_b200.utils.microbench peers_step --mode fp32_master --elems 67108864 --world 8
    python -m offload_adam_b200.utils.microbench peer_reduce --elems 67108864 --world 8
    python -m offload_adam_b200.utils.microbench multi_tensor --tensors 65 --elems 4096

Each case warms up, then times ``--iters`` launches with CUDA events on the launching
stream (operands are far larger than L2 unless ``--elems`` is made small), and prints one
JSON line with the algorithmic bytes, the achieved GB/s and the fraction of the measured
peak (``MEASURED_PEAKS.json`` at the repository root when present, else the documented
fallback of 6650 GB/s for HBM; PCIe cases are compared with a full-duplex
``cudaMemcpyAsync`` measured in the same run).  Small ``--elems`` make the cases suitable
for an ``ncu`` capture of a single launch.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

BYTES_PER_ELEM = {"stochastic_rounding": 14, "fp32_master": 20, "fp31_master": 18,
                  "fp32_master_custom_rounding": 18}


def hbm_peak_gbs():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        return json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["hbm_gbs"], "measured"
    except Exception:
        return 6650.0, "fallback"


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return min(times), sum(times) / len(times)


def make_states(n, mode, device):
    st = {"grad": (torch.randn(n, device=device) * 1e-2).to(torch.bfloat16),
          "exp_avg": torch.zeros(n, dtype=torch.bfloat16, device=device),
          "exp_avg_sq": torch.zeros(n, dtype=torch.bfloat16, device=device)}
    p = (torch.randn(n, device=device) * 0.02).to(torch.bfloat16)
    if mode == "fp32_master":
        st["master_params"] = p.float()
    elif mode != "stochastic_rounding":
        st["rounding_error"] = torch.zeros(n, dtype=torch.int16, device=device)
    return p, st


def case_adam_step(args):
    from ..ops.adam_step import adam_step
    p, st = make_states(args.elems, args.mode, "cuda")
    step = [1]

    def run():
        step[0] += 1
        adam_step(args.mode, p, st, 1e-4, 0.01, 0.9, 0.999, 1e-8, step[0], decoupled_weight_decay=True, seed=1)

    best, avg = timeit(run, args.iters)
    nbytes = args.elems * BYTES_PER_ELEM[args.mode]
    peak, src = hbm_peak_gbs()
    return {"case": "adam_step", "mode": args.mode, "elems": args.elems, "ms": best, "ms_avg": avg,
            "bytes": nbytes, "GBs": nbytes / best / 1e6, "peak_GBs": peak,
            "fraction_of_%s_hbm_copy" % src: nbytes / best / 1e6 / peak}


def case_peers_step(args):
    """The fused pull + average + Adam + push kernel of the ZeRO-1 path on ONE GPU: the
    replicas of the other ranks are buffers of the same device (the kernel only sees
    addresses), so the traffic that would cross NVLink stays in HBM.  Useful for an
    ``ncu`` capture of the kernel and as an upper bound of its rate."""
    from ..ops.adam_step import adam_step
    n, w = args.elems, args.world
    p, st = make_states(n, args.mode, "cuda")
    st.pop("grad")
    grads = [(torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16) for _ in range(w)]
    replicas = [p] + [torch.empty_like(p) for _ in range(w - 1)]
    step = [1]

    def run():
        step[0] += 1
        adam_step(args.mode, p, st, 1e-4, 0.01, 0.9, 0.999, 1e-8, step[0], decoupled_weight_decay=True, seed=1,
                  g_peers=[g.data_ptr() for g in grads], g_scale=1.0 / w,
                  p_peers=[r.data_ptr() for r in replicas])

    best, avg = timeit(run, args.iters)
    # per element: w gradients read, state read and written, w parameter replicas written
    nbytes = n * (BYTES_PER_ELEM[args.mode] - 4 + 2 * w + 2 * w)
    peak, src = hbm_peak_gbs()
    return {"case": "peers_step", "mode": args.mode, "elems": n, "world": w, "ms": best, "ms_avg": avg,
            "bytes": nbytes, "GBs": nbytes / best / 1e6, "peak_GBs": peak,
            "fraction_of_%s_hbm_copy" % src: nbytes / best / 1e6 / peak}


def case_accumulate(args):
    from ..ops import grad_ops
    a = torch.randn(args.elems, device="cuda").to(torch.bfloat16)
    b = torch.randn(args.elems, device="cuda").to(torch.bfloat16)
    sq = torch.zeros(1, device="cuda")
    scratch = grad_ops.sumsq_scratch("cuda")
    best, avg = timeit(lambda: grad_ops.grad_accumulate(a, a, b, sumsq=sq, scratch=scratch), args.iters)
    nbytes = args.elems * 6
    peak, src = hbm_peak_gbs()
    return {"case": "accumulate+sumsq", "elems": args.elems, "ms": best, "bytes": nbytes,
            "GBs": nbytes / best / 1e6, "fraction_of_%s_hbm_copy" % src: nbytes / best / 1e6 / peak}


def duplex_memcpy_gbs(nbytes):
    host_a = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    host_b = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dev_a = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    dev_b = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def run():
        cur = torch.cuda.current_stream()
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        with torch.cuda.stream(s1):
            dev_a.copy_(host_a, non_blocking=True)
        with torch.cuda.stream(s2):
            host_b.copy_(dev_b, non_blocking=True)
        cur.wait_stream(s1)
        cur.wait_stream(s2)

    best, _ = timeit(run, 3, warmup=1)
    return nbytes / best / 1e6


def case_staged_step(args):
    from ..engine import TransferEngine
    from .pinned_alloc import PinnedArena
    n, mode = args.elems, args.mode
    specs = [((n,), torch.bfloat16), ((n,), torch.bfloat16)]
    if mode == "fp32_master":
        specs.append(((n,), torch.float32))
    elif mode != "stochastic_rounding":
        specs.append(((n,), torch.int16))
    arena = PinnedArena(specs, numa_node="auto")
    ts = list(arena.tensors())
    states = {"exp_avg": ts[0], "exp_avg_sq": ts[1]}
    if mode == "fp32_master":
        states["master_params"] = ts[2]
    elif mode != "stochastic_rounding":
        states["rounding_error"] = ts[2]
    p = (torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16)
    g = (torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16)
    eng = TransferEngine("cuda", mode, 1, transfer=args.transfer, chunk_elems=args.chunk_elems,
                         ring_slots=args.ring_slots)
    step = [1]

    def run():
        step[0] += 1
        eng.step(0, p, g, None, states, (1e-4, 0.01, 0.9, 0.999, 1e-8), step[0], True, seed=1)
        eng.join_main()

    best, avg = timeit(run, args.iters, warmup=1)
    each_way = n * (BYTES_PER_ELEM[mode] - 6)  # state bytes moved per direction
    link = duplex_memcpy_gbs(min(each_way, 1 << 30))
    return {"case": "staged_step", "transfer": eng.transfer, "mode": mode, "elems": n, "ms": best,
            "bytes_each_direction": each_way, "GBs_each_direction": each_way / best / 1e6,
            "duplex_memcpy_GBs_each_direction": link,
            "fraction_of_measured_duplex_memcpy": each_way / best / 1e6 / link,
            "arena": arena.stats()}


def _quant_classes(impl):
    if impl == "reference":
        import sys
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        ref = os.path.join(root, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref, "offload_adam")):
            raise SystemExit("the reference package is not installed under baseline/_ref")
        if ref not in sys.path:
            sys.path.insert(0, ref)
        from offload_adam import qweight as q
    else:
        from .. import qweight as q
    return {"nvfp4": q.NVFP4QWeight, "nf4": q.NF4QWeight, "int4": q.Int4QWeight, "int8": q.Int8QWeight}


def case_quant(args):
    """Quantize (``copy_`` of a dense tensor into the packed weight), de-quantize and, for
    this package, the one-pass fake quantization; ``--impl reference`` times the reference
    package's Triton kernels through the same calls."""
    cls = _quant_classes(args.impl)[args.format]
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[args.input_dtype]
    src = (torch.randn(args.rows, args.cols, device="cuda") * 0.02).to(dtype)
    q = cls.from_float(torch.zeros(args.rows, args.cols, dtype=torch.bfloat16, device="cuda"))
    tq, _ = timeit(lambda: q.copy_(src), args.iters)
    td, _ = timeit(lambda: q.dequantize(torch.bfloat16), args.iters)
    n = args.rows * args.cols
    packed = sum(t.numel() * t.element_size() for t in (q._payload() if hasattr(q, "_payload") else
                                                        [getattr(q, k) for k in q.__tensor_flatten__()[0]]))
    peak, src_name = hbm_peak_gbs()
    eb = src.element_size()
    out = {"case": "quant", "impl": args.impl, "format": args.format, "shape": [args.rows, args.cols],
           "input": args.input_dtype,
           "quantize_ms": tq, "quantize_GBs": (eb * n + packed) / tq / 1e6,
           "quantize_fraction_of_%s_hbm_copy" % src_name: (eb * n + packed) / tq / 1e6 / peak,
           "dequantize_ms": td, "dequantize_GBs": (2 * n + packed) / td / 1e6,
           "dequantize_fraction_of_%s_hbm_copy" % src_name: (2 * n + packed) / td / 1e6 / peak,
           "note": "bytes are the algorithmic ones: input once, payload once (NVFP4 also reads the input once "
                   "more for the tensor maximum, which is not counted)"}
    if args.impl == "ours":
        from ..qweight import fake_quantize
        x16 = src.to(torch.bfloat16)
        tf, _ = timeit(lambda: fake_quantize(x16, cls), args.iters)
        out.update(fake_quant_ms=tf, fake_quant_GBs=4 * n / tf / 1e6)
    return out


def case_quant_table(args):
    """All formats x two weight shapes of the 8B model x fp32 (master) and bf16 input, this
    package and (when installed) the reference.  One JSON line per row."""
    rows = []
    impls = ["ours"]
    try:
        _quant_classes("reference")
        impls.append("reference")
    except SystemExit:
        pass
    for shape in ((4096, 14336), (128256, 4096)):
        for fmt in ("nvfp4", "nf4", "int4", "int8"):
            for dt in ("fp32", "bf16"):
                for impl in impls:
                    a = argparse.Namespace(**vars(args))
                    a.rows, a.cols, a.format, a.input_dtype, a.impl = shape[0], shape[1], fmt, dt, impl
                    try:
                        r = case_quant(a)
                    except Exception as e:  # a reference kernel that does not take the case
                        r = {"case": "quant", "impl": impl, "format": fmt, "shape": list(shape), "input": dt,
                             "error": repr(e)[:200]}
                    print(json.dumps(r), flush=True)
                    rows.append(r)
                    torch.cuda.empty_cache()
    return {"case": "quant_table", "rows": len(rows)}


def case_adam_quant(args):
    """The fused step of a quantized weight (Adam on the fp32 master + re-quantize + store of
    the packed rows into ``--world`` replicas) on ONE GPU: the other ranks' payloads are
    buffers of the same device.  NVFP4 runs its two passes (step with max|master| and a
    device copy of the master, then quantize + push)."""
    from .. import _ext
    from ..ops.oracle import beta_hat
    C = _ext.load(required=True)
    rows, cols, w = args.rows, args.cols, args.world
    n = rows * cols
    master = torch.randn(rows, cols, device="cuda") * 0.02
    g = (torch.randn(rows, cols, device="cuda") * 1e-2).to(torch.bfloat16)
    m = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    fmt = args.format
    fid = {"nvfp4": C.QFMT_NVFP4, "nf4": C.QFMT_NF4, "int4": C.QFMT_INT4, "int8": C.QFMT_INT8}[fmt]
    group = {"nvfp4": 16, "nf4": 64, "int4": 128, "int8": 0}[fmt]
    if fmt in ("nvfp4", "nf4"):
        pay = [(torch.empty(rows, cols // 2, dtype=torch.uint8, device="cuda"),
                torch.empty(n // group * (4 if fmt == "nf4" else 1), dtype=torch.uint8, device="cuda")) for _ in range(w)]
    elif fmt == "int4":
        pay = [(torch.empty(cols // 8, rows, dtype=torch.int32, device="cuda"),
                torch.empty(cols // group, rows, dtype=torch.bfloat16, device="cuda")) for _ in range(w)]
    else:
        pay = [(torch.empty(rows, cols, dtype=torch.int8, device="cuda"),
                torch.empty(rows, dtype=torch.bfloat16, device="cuda")) for _ in range(w)]
    amax = torch.zeros(1, device="cuda")
    gs = torch.zeros((), device="cuda")
    copy = torch.empty_like(master) if fmt == "nvfp4" else None
    spec = C.QuantSpec(fid, rows, cols, 0, group, C.QDT_BF16, [a.data_ptr() for a, _ in pay],
                       [b.data_ptr() for _, b in pay], amax if fmt == "nvfp4" else None, gs if fmt == "nvfp4" else None)
    step = [1]

    def run():
        step[0] += 1
        b1, b2 = beta_hat(0.9, step[0]), beta_hat(0.999, step[0])
        if fmt == "nvfp4":
            amax.zero_()
            C.adam_step(1, None, g, None, m, v, master, 1e-4, 0.01, b1, b2, 1e-8, True, None, 0, 0, amax, 0, 0,
                        [], 1.0, [], None, copy)
            C.nvfp4_quantize_push(spec, copy.data_ptr(), n, None, 0)
        else:
            C.adam_quant_push(spec, g, None, m, v, master, 1e-4, 0.01, b1, b2, 1e-8, True, None, 0, 0, [], 1.0, None)

    best, avg = timeit(run, args.iters)
    packed = sum(a.numel() * a.element_size() + b.numel() * b.element_size() for a, b in pay[:1])
    nbytes = n * (2 + 4 + 4 + 8) + packed * w + (8 * n if fmt == "nvfp4" else 0)
    peak, src = hbm_peak_gbs()
    return {"case": "adam_quant", "format": fmt, "shape": [rows, cols], "world": w, "ms": best, "ms_avg": avg,
            "bytes": nbytes, "GBs": nbytes / best / 1e6, "fraction_of_%s_hbm_copy" % src: nbytes / best / 1e6 / peak}


def case_peer_reduce(args):
    """Pull + average (+ squared norm) of the ZeRO-1 clip path with same-device replicas."""
    from .. import _ext
    from ..ops import grad_ops
    C = _ext.load(required=True)
    n, w = args.elems, args.world
    grads = [(torch.randn(n, device="cuda") * 1e-2).to(torch.bfloat16) for _ in range(w)]
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    sq = torch.zeros(1, device="cuda")
    scratch = grad_ops.sumsq_scratch("cuda")
    ptrs = [g.data_ptr() for g in grads]
    best, avg = timeit(lambda: C.peer_reduce(out, ptrs, 1.0 / w, sq, scratch, None, 0, 0), args.iters)
    nbytes = n * 2 * (w + 1)
    peak, src = hbm_peak_gbs()
    return {"case": "peer_reduce+sumsq", "elems": n, "world": w, "ms": best, "bytes": nbytes,
            "GBs": nbytes / best / 1e6, "fraction_of_%s_hbm_copy" % src: nbytes / best / 1e6 / peak}


def case_multi_tensor(args):
    """One launch that steps every small GPU-resident tensor (latency-bound)."""
    from ..ops import grad_ops
    entries = []
    for _ in range(args.tensors):
        p, st = make_states(args.elems, args.mode, "cuda")
        entries.append({"param": p, "grad": st["grad"], "exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"],
                        "extra": st.get("master_params", st.get("rounding_error")), "p": p})
    mt = grad_ops.MultiTensorAdam(entries, args.mode)
    step = [1]

    def run():
        step[0] += 1
        mt.step(1e-4, 0.01, 0.9, 0.999, 1e-8, step[0], True, seed=1, zero_grad=False)

    best, avg = timeit(run, args.iters)
    nbytes = args.tensors * args.elems * BYTES_PER_ELEM[args.mode]
    return {"case": "multi_tensor_adam", "mode": args.mode, "tensors": args.tensors, "elems_each": args.elems,
            "ms": best, "ms_avg": avg, "bytes": nbytes, "GBs": nbytes / best / 1e6}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["adam_step", "peers_step", "accumulate", "staged_step", "quant", "quant_table",
                                     "adam_quant", "peer_reduce", "multi_tensor"])
    ap.add_argument("--mode", default="fp32_master", choices=list(BYTES_PER_ELEM))
    ap.add_argument("--elems", type=int, default=256 << 20)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--transfer", default="staged", choices=["staged", "zero_copy"])
    ap.add_argument("--chunk-elems", type=int, default=8 << 20)
    ap.add_argument("--ring-slots", type=int, default=4)
    ap.add_argument("--world", type=int, default=8, help="peers_step: number of (same-device) replicas")
    ap.add_argument("--format", default="nvfp4", choices=["nvfp4", "nf4", "int4", "int8"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--input-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--tensors", type=int, default=65)
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--cols", type=int, default=4096)
    args = ap.parse_args()
    fn = {"adam_step": case_adam_step, "peers_step": case_peers_step, "accumulate": case_accumulate, "staged_step": case_staged_step,
          "quant": case_quant, "quant_table": case_quant_table, "adam_quant": case_adam_quant,
          "peer_reduce": case_peer_reduce, "multi_tensor": case_multi_tensor}[args.case]
    print(json.dumps(fn(args)))


if __name__ == "__main__":
    main()
