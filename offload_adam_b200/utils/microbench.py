"""Kernel micro-benchmarks with roofline fractions.

    python -m offload_adam_b200.utils.microbench adam_step --mode fp32_master --elems 268435456
    python -m offload_adam_b200.utils.microbench staged_step --mode fp32_master --elems 134217728
    python -m offload_adam_b200.utils.microbench accumulate --elems 268435456
    python -m offload_adam_b200.utils.microbench quant --format nvfp4 --rows 14336 --cols 4096
    python -m offload_adam_b200.utils.microbench peers_step --mode fp32_master --elems 67108864 --world 8

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


def case_quant(args):
    from ..qweight import Int4QWeight, Int8QWeight, NF4QWeight, NVFP4QWeight
    cls = {"nvfp4": NVFP4QWeight, "nf4": NF4QWeight, "int4": Int4QWeight, "int8": Int8QWeight}[args.format]
    master = torch.randn(args.rows, args.cols, device="cuda") * 0.02
    q = cls.from_float(torch.zeros(args.rows, args.cols, dtype=torch.bfloat16, device="cuda"))
    tq, _ = timeit(lambda: q.copy_(master), args.iters)
    td, _ = timeit(lambda: q.dequantize(torch.bfloat16), args.iters)
    n = args.rows * args.cols
    packed = sum(t.numel() * t.element_size() for t in q._payload())
    peak, src = hbm_peak_gbs()
    amax_pass = 4 * n if args.format == "nvfp4" else 0  # tensor amax needs its own read
    return {"case": "quant", "format": args.format, "shape": [args.rows, args.cols],
            "quantize_ms": tq, "quantize_GBs": (4 * n + packed + amax_pass) / tq / 1e6,
            "dequantize_ms": td, "dequantize_GBs": (2 * n + packed) / td / 1e6,
            "peak_GBs(%s)" % src: peak}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["adam_step", "peers_step", "accumulate", "staged_step", "quant"])
    ap.add_argument("--mode", default="fp32_master", choices=list(BYTES_PER_ELEM))
    ap.add_argument("--elems", type=int, default=256 << 20)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--transfer", default="staged", choices=["staged", "zero_copy"])
    ap.add_argument("--chunk-elems", type=int, default=8 << 20)
    ap.add_argument("--ring-slots", type=int, default=4)
    ap.add_argument("--world", type=int, default=8, help="peers_step: number of (same-device) replicas")
    ap.add_argument("--format", default="nvfp4", choices=["nvfp4", "nf4", "int4", "int8"])
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--cols", type=int, default=4096)
    args = ap.parse_args()
    fn = {"adam_step": case_adam_step, "peers_step": case_peers_step, "accumulate": case_accumulate, "staged_step": case_staged_step,
          "quant": case_quant}[args.case]
    print(json.dumps(fn(args)))


if __name__ == "__main__":
    main()
