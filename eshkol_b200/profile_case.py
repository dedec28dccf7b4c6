"""Run one GEMM shape on device-resident operands and print per-stage times.

    python -m eshkol_b200.profile_case --n 4096 --tier exact --reps 3

The counterpart of the reference's ESHKOL_OZAKI_PROFILE line
(lib/backend/gpu/gpu_memory.mm:2658-2664): milliseconds per stage and
f64-equivalent GFLOP/s of the whole product.  Small enough to sit under a profiler.
"""
from __future__ import annotations

import argparse
import ctypes
import json

import eshkol_b200 as eb
from eshkol_b200 import api, inputs

TIERS = {"exact": eb.TIER_OZAKI2, "ozaki1": eb.TIER_OZAKI1, "fast": eb.TIER_OZAKI2_FAST, "dgemm": eb.TIER_DGEMM}
STAGES = ["scan_b", "split_b", "scan_a", "split_a", "products_mod256", "products_odd", "reconstruct"]


def main() -> None:
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--m", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--tier", default="exact", choices=sorted(TIERS) + ["f16"],
                    help="f16: the half-precision dtype path (f64 storage, f16 operands, f32 accumulation)")
    ap.add_argument("--param", type=int, default=0)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--tile-n", type=int, default=0, choices=[0, 128, 256])
    ap.add_argument("--pair", type=int, default=-1, help="1: two-SM products kernel, 0: one-SM")
    ap.add_argument("--band-rows", type=int, default=-1, help="rows per band of the row-band pipeline, 0: off")
    ap.add_argument("--dist", default="normal", choices=["normal", "uniform", "wide"])
    args = ap.parse_args()
    M, K, N = args.m or args.n, args.k or args.n, args.n
    dev = torch.device("cuda", 0)
    gen = getattr(inputs, args.dist)
    A = gen(1, (M, K), device=dev)
    B = gen(2, (K, N), device=dev)
    C = torch.empty((M, N), dtype=torch.float64, device=dev)
    torch.cuda.synchronize()
    lib = eb.load_library()
    if lib.eshkol_b200_init(0) != 0:
        raise RuntimeError("no usable sm_100 device")
    lib.eshkol_b200_set_phase_timing(1)
    if args.pair >= 0:
        lib.eshkol_b200_set_pair_gemm(args.pair)
    if args.band_rows >= 0:
        lib.eshkol_b200_set_row_bands(args.band_rows)
    opts = api.make_opts(TIERS.get(args.tier, 0), args.param, tile_n=args.tile_n)
    stream = torch.cuda.ExternalStream(api.stream_handle(), device=dev)
    out = {}
    for rep in range(args.reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if args.tier == "f16":
            if lib.eshkol_b200_gemm_f16_device(A.data_ptr(), B.data_ptr(), C.data_ptr(), 1, M, K, N) != 0:
                raise RuntimeError("gemm_f16 failed")
        else:
            api.gemm_device(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, K, N, opts)
        e1.record(stream)
        if api.sync_status() != 0:
            raise RuntimeError("kernel status non-zero")
        ms = e0.elapsed_time(e1)
        out = {"M": M, "K": K, "N": N, "tier": args.tier, "ms": ms,
               "gflops_f64_equivalent": 2.0 * M * K * N / ms / 1e6}
        if args.tier == "exact":
            ph = (ctypes.c_float * 8)()
            if lib.eshkol_b200_get_phase_times(ph, 8) == 7:
                out["stages_ms"] = dict(zip(STAGES, (round(float(x), 4) for x in ph[:7])))
                out["bands"] = int(ph[7])
    print(json.dumps(out))


if __name__ == "__main__":
    main()
