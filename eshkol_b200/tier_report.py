"""Throughput and error of every precision tier on one shape (default 8192^3, normal entries).

    python -m eshkol_b200.tier_report --n 8192

For each tier: f64-equivalent TFLOP/s on device-resident operands (CUDA events on the
library stream, best and median of the timed repetitions) and the error on the same
operands against two references: the exact tier's result (the reference's arithmetic,
whose CRT accumulation itself rounds in a fraction of the cells) and the 16-moduli fast
tier (integer CRT, no rounding before the final conversion: the most accurate result the
library produces).  Errors are the maximum element-wise relative error with the
denominator rule of the reference's probes (|ref| > 1e-9 ? |ref| : 1,
tests/gpu/ozaki_correctness_test.esk:64-65) and the normwise Frobenius error
(tests/gpu/cuda_ozaki_correctness_test.esk:46-72).  One JSON line per tier.
"""
from __future__ import annotations

import argparse
import json

import eshkol_b200 as eb
from eshkol_b200 import api, inputs

TIERS = [("ozaki2-exact-16", eb.TIER_OZAKI2, 16), ("ozaki2-fast-16", eb.TIER_OZAKI2_FAST, 16)]
TIERS += [(f"ozaki2-fast-{n}", eb.TIER_OZAKI2_FAST, n) for n in (10, 11, 12, 14)]
TIERS += [(f"ozaki1-T{t}", eb.TIER_OZAKI1, t) for t in (1, 2, 3, 4, 5, 6, 7)]
TIERS += [("native-f64-cuda-cores", eb.TIER_DGEMM, 0)]


def main() -> None:
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--dist", default="normal", choices=["normal", "uniform", "wide"])
    args = ap.parse_args()
    n = args.n
    dev = torch.device("cuda", 0)
    gen = getattr(inputs, args.dist)
    A = gen(1, (n, n), device=dev)
    B = gen(2, (n, n), device=dev)
    torch.cuda.synchronize()
    lib = eb.load_library()
    if lib.eshkol_b200_init(0) != 0:
        raise RuntimeError("no usable sm_100 device")
    stream = torch.cuda.ExternalStream(api.stream_handle(), device=dev)
    ref = None   # exact tier
    best = None  # fast tier, 16 moduli

    def errors(C, R):
        diff = (C - R).abs()
        denom = torch.where(R.abs() > 1e-9, R.abs(), torch.ones_like(R))
        return float((diff / denom).max()), float(torch.linalg.norm(C - R) / torch.linalg.norm(R))

    for name, tier, param in TIERS:
        C = torch.empty((n, n), dtype=torch.float64, device=dev)
        opts = api.make_opts(tier, param)
        reps = 1 if tier == eb.TIER_DGEMM else args.reps
        times = []
        for rep in range(reps + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            api.gemm_device(A.data_ptr(), B.data_ptr(), C.data_ptr(), n, n, n, opts)
            e1.record(stream)
            if api.sync_status() != 0:
                raise RuntimeError("kernel status non-zero")
            if rep > 0 or reps == 1:
                times.append(e0.elapsed_time(e1))
        times.sort()
        out = {"tier": name, "n": n, "ms_best": times[0], "ms_median": times[len(times) // 2],
               "tflops_f64_equivalent": 2.0 * n ** 3 / times[len(times) // 2] / 1e9}
        if ref is None:
            ref = C
        elif best is None:
            best = C
            e = errors(ref, best)
            print(json.dumps({"note": "exact tier measured against the 16-moduli fast tier",
                              "max_rel_err": e[0], "normwise_err": e[1]}), flush=True)
        out["max_rel_err_vs_exact_tier"], out["normwise_err_vs_exact_tier"] = errors(C, ref)
        if best is not None:
            out["max_rel_err_vs_fast16"], out["normwise_err_vs_fast16"] = errors(C, best)
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
