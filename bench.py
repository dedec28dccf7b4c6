#!/usr/bin/env python
"""Benchmark of the f64 GEMM hot path (Ozaki-II exact tier).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N = 1: 8192^3, standard-normal operands, exact tier (the single-GPU configuration
the headline metric is quoted on).  N > 1 (launched under torch.distributed.run):
32768^3, uniform[-1,1) operands, rows of A sharded across the ranks, B broadcast
from rank 0 and C all-gathered over NCCL, all inside the timed step.
One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "f64-equivalent TFLOP/s, Ozaki-II exact GEMM"
UNIT = "TFLOP/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region (read-only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            parts = [p.strip() for p in r.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        # the busy half of the samples: idle samples before/after the loop would pull the median down
        busy = sm[len(sm) // 2:] if sm else []
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ reference arm
def cpu_reference_run(n_full: int, rows: int, steps: int, warmup: int, dist_name: str):
    """The reference's own CPU matmul (eshkol_matmul_f64, lib/backend/blas_backend.cpp:791)
    on a slab of `rows` rows of the n_full^3 product."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    from eshkol_b200 import inputs
    gen = inputs.normal if dist_name == "normal" else inputs.uniform
    A = gen(1, (rows, n_full))
    B = gen(2, (n_full, n_full))
    kind, cores, fn = "reference", os.cpu_count() or 1, None
    if ol.ref_lib("libref_matmul_blas.so") is not None:
        os.environ.setdefault("OPENBLAS_NUM_THREADS", str(cores))
        fn = lambda: ol.ref_matmul(A, B, blas=True)
        how = "eshkol_matmul_f64 -> cblas_dgemm (OpenBLAS bundled in the image)"
    elif ol.ref_lib("libref_matmul_simd.so") is not None:
        fn, cores = (lambda: ol.ref_matmul(A, B, blas=False)), 1
        how = "eshkol_matmul_f64 -> matmul_simd_avx (single thread by construction)"
    else:
        kind, cores = "port", os.cpu_count() or 1
        sub = min(rows, 64)
        A = A[:sub]
        rows = sub
        fn = lambda: ol.oz2_exact(A, B, 52)
        how = "oracle restatement of the exact tier (OpenMP)"
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * rows * n_full * n_full / dt / 1e12
    return {"value": tflops, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{rows} rows of the {n_full}^3 product, {steps} timed passes; {how}"}, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = 8192 if args.gpus == 1 else 32768
    dist_name = "normal" if args.gpus == 1 else "uniform"
    rows = 1024 if n == 8192 else 128
    base, dt = cpu_reference_run(n, rows, max(1, args.steps), max(1, min(args.warmup, 2)), dist_name)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, panels: int = 0):
    if n_gpus == 1:
        return {"workload": "f64 GEMM 8192x8192x8192, exact (Ozaki-II, 16 moduli) tier, entries standard normal "
                            "(48-bit LCG + Box-Muller), single B200", "M": 8192, "K": 8192, "N": 8192,
                "l2": "operands (512 MiB each) exceed the 126 MB L2; no explicit flush"}
    return {"workload": "f64 GEMM 32768x32768x32768, exact tier, entries uniform[-1,1), rows of A sharded across "
                        f"{n_gpus} B200, B distributed from rank 0 and C gathered on every rank over NVLink inside the step",
            "M": 32768, "K": 32768, "N": 32768, "parallelism": f"row-shard x{n_gpus}",
            "l2": "operands exceed the 126 MB L2; no explicit flush"}


# ----------------------------------------------------------------------- our arm
def run_b200(args):
    import numpy as np
    import torch
    import eshkol_b200 as eb
    from eshkol_b200 import api, inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    comm_sms = int(os.environ.get("ESHKOL_B200_COMM_SMS", "0"))  # measured: capping the collectives' CTAs costs more than it frees
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        if comm_sms > 0:
            # the collectives run on the SMs the products kernels leave free (see ShardedGemm)
            os.environ.setdefault("NCCL_MAX_CTAS", str(comm_sms))
        dist.init_process_group("nccl", device_id=dev)
    api.set_device(local)
    lib = eb.load_library()
    if lib.eshkol_b200_init(local) != 0:
        raise RuntimeError("eshkol_b200_init failed: this benchmark has no fallback path")
    lib_stream = torch.cuda.ExternalStream(api.stream_handle(), device=dev)

    n = 8192 if world == 1 else 32768
    opts = api.make_opts(eb.TIER_OZAKI2, 16)
    if world == 1:
        rows = n
        A = inputs.normal(1, (n, n), device=dev)
        B = inputs.normal(2, (n, n), device=dev)
        C_local = torch.empty((n, n), dtype=torch.float64, device=dev)
        sg = None
    else:
        from eshkol_b200.sharded import ShardedGemm
        # column panels of B overlap the broadcast and the gather with the products; worth it
        # once the collectives are a visible share of the step (4 ranks and more)
        panels = int(os.environ.get("ESHKOL_B200_PANELS", "4"))
        transport = os.environ.get("ESHKOL_B200_TRANSPORT", "copy_engine")
        # a first and a last panel of half the width shorten the two transfers nothing hides
        taper = os.environ.get("ESHKOL_B200_TAPER", "1") == "1"
        sg = ShardedGemm(n, n, n, dev, tier=eb.TIER_OZAKI2, param=16, panels=panels, comm_sms=comm_sms,
                         transport=transport, taper=taper)
        rows = sg.rows
        A = inputs.uniform(1, (rows, n), device=dev, start=sg.row0 * n)
        B = inputs.uniform(2, (n, n), device=dev) if rank == 0 else None
        C_local = torch.empty((rows, sg.width), dtype=torch.float64, device=dev)  # the stage-timed product's output
    torch.cuda.synchronize()

    def step():
        if sg is None:
            api.gemm_device(A.data_ptr(), B.data_ptr(), C_local.data_ptr(), n, n, n, opts)
        else:
            sg.step(A, B)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if api.sync_status() != 0:
            raise RuntimeError("kernel status non-zero")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    # clock soak: nvidia-smi samples every 100 ms and K steps can be shorter than that, so the
    # same step is repeated untimed, directly before the timed region, until about 1.2 s of
    # samples exist (a fixed count when sharded); the GPU enters the timed region in the power / thermal state they show
    soak_steps = 0
    if world == 1:
        t_soak = time.perf_counter()
        while time.perf_counter() - t_soak < 1.2 and soak_steps < 400:
            for _ in range(4):
                step()
                soak_steps += 1
            torch.cuda.synchronize()
    else:
        # every rank must run the same number of collective steps: a fixed count (a step of
        # the sharded configuration takes 0.09 - 0.26 s)
        for _ in range(8):
            step()
            soak_steps += 1
    barrier()
    lib.eshkol_b200_set_phase_timing(1)
    launches0 = api.launch_count()
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)
    barrier()
    if world == 1:
        ev0.record(lib_stream)
        for _ in range(args.steps):
            step()
        ev1.record(lib_stream)
        barrier()
        ms_total = ev0.elapsed_time(ev1)
    else:
        # the step mixes the library stream and torch's (NCCL) stream with host waits in
        # between: bracket it with events on torch's stream after a full device sync
        ev0.record(torch.cuda.current_stream())
        for _ in range(args.steps):
            step()
        torch.cuda.current_stream().synchronize()
        ev1.record(torch.cuda.current_stream())
        barrier()
        ms_total = ev0.elapsed_time(ev1)
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    launches = api.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = f"{soak_steps} identical untimed steps directly before + the {args.steps} timed steps"
    ms_step = ms_total / args.steps
    value = 2.0 * n * n * n / (ms_step * 1e-3) / 1e12

    # per-stage times of one more (untimed) GEMM, for the roofline of the dominant kernel
    ph = (ctypes.c_float * 8)()
    Bdev = B if sg is None else sg.Bp[sg.panels // 2]  # a full-width panel when the edge panels are halved
    api.gemm_device(A.data_ptr(), Bdev.data_ptr(), C_local.data_ptr(), rows, n, Bdev.shape[1], opts)
    got = lib.eshkol_b200_get_phase_times(ph, 8)
    lib.eshkol_b200_set_phase_timing(0)
    phases = [float(x) for x in ph[:7]] if got == 7 else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # sharded run: rows another rank computed and this rank only received must carry the bits
    # of the same rows multiplied here
    verified = None
    if sg is not None:
        r_last, _ = sg.parts[world - 1]
        probe = 128
        A_probe = inputs.uniform(1, (probe, n), device=dev, start=r_last * n)
        C_probe = torch.empty((probe, n), dtype=torch.float64, device=dev)
        torch.cuda.synchronize()
        api.gemm_device(A_probe.data_ptr(), B.data_ptr(), C_probe.data_ptr(), probe, n, n, opts)
        if api.sync_status() != 0:
            raise RuntimeError("kernel status non-zero")
        if not torch.equal(C_probe.view(torch.int64), sg.C[r_last:r_last + probe].view(torch.int64)):
            raise RuntimeError("gathered rows differ from the same rows multiplied on one GPU")
        verified = probe
        del A_probe, C_probe

    peaks = measured_peaks()
    roofline = None
    if phases:
        t_odd = phases[5] * 1e-3
        ops = 15 * 2.0 * rows * n * Bdev.shape[1]  # 15 odd-modulus int8 GEMMs (one column panel when sharded)
        achieved = ops / t_odd / 1e12
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        roofline = {
            "kernel": "modgemm_kernel<256, odd moduli> (tcgen05 int8 -> int32, 15 planes)",
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "traffic": None,
            "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}); "
                           "int8 dense issues at twice the bf16 rate",
            "phases_ms": dict(zip(["scan_b", "split_b", "scan_a", "split_a", "products_mod256",
                                   "products_odd", "reconstruct"], phases)),
        }
        # the memory-side stages against the measured copy bandwidth: algorithmic bytes per
        # element are 8 read + 15 (odd planes) + 1024/1008 (modulus-256 plane) + 0.25 (flag
        # bit-planes) written for a split, 15 + 2 + 0.125 read + 8 written for the reconstruction
        kn = float(n) * Bdev.shape[1]
        mk = float(rows) * n
        mn = float(rows) * Bdev.shape[1]
        split_bytes = 8.0 + 15.0 + 1024.0 / 1008.0 + 0.25
        stages = [("scan_cols (B)", 8.0 * kn, phases[0]), ("split_b", split_bytes * kn, phases[1]),
                  ("scan_rows (A)", 8.0 * mk, phases[2]), ("split_a", split_bytes * mk, phases[3]),
                  ("crt (reconstruction)", (17.125 + 8.0) * mn, phases[6])]
        roofline["hbm_stages"] = [
            {"kernel": name, "bound": "hbm", "achieved": b / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
             "unit": "GB/s", "frac": b / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "ms": ms}
            for name, b, ms in stages if ms > 0]
        int8_peak = measure_int8_library_peak(torch, dev)
        if int8_peak:
            roofline["int8_cublaslt_tops_live"] = int8_peak
            roofline["frac_of_int8_library"] = achieved / int8_peak
        fp64 = measure_fp64_library_peak(torch, dev)
        if fp64:
            roofline["native_fp64_gemm_tflops_live"] = fp64
            roofline["value_vs_native_fp64"] = value / fp64

    # end to end through the reference-facing dispatcher, host buffers in pinned memory
    e2e = None
    if world == 1:
        hA = torch.empty((n, n), dtype=torch.float64).pin_memory()
        hB = torch.empty((n, n), dtype=torch.float64).pin_memory()
        hC = torch.empty((n, n), dtype=torch.float64).pin_memory()
        hA.copy_(A)
        hB.copy_(B)
        torch.cuda.synchronize()
        lib.eshkol_gpu_init()
        e2e_steps = max(2, min(args.steps, 5))
        for _ in range(2):
            lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
        dt = (time.perf_counter() - t0) / e2e_steps
        e2e = {"value": 2.0 * n * n * n / dt / 1e12, "unit": UNIT, "h2d_bytes_per_step": 2 * n * n * 8,
               "d2h_bytes_per_step": n * n * 8, "ms_per_step": dt * 1e3,
               "api": "eshkol_matmul_dispatch(host A, host B, host C), pinned host memory"}
    else:
        e2e = {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "sharded configuration is defined on device-resident operands; see the 1-GPU line for PCIe"}

    # The sharded configuration on this one GPU (it fits: about 90 GB): the denominator for the
    # parallel efficiency of the 2 / 4 / 8-GPU lines, whose workload it is.
    one_gpu_sharded_shape = None
    if world == 1 and os.environ.get("ESHKOL_B200_SKIP_32768", "") != "1":
        try:
            del A, B, C_local
            if e2e is not None:
                del hA, hB, hC
            torch.cuda.empty_cache()
            nn = 32768
            A32 = inputs.uniform(1, (nn, nn), device=dev)
            B32 = inputs.uniform(2, (nn, nn), device=dev)
            C32 = torch.empty((nn, nn), dtype=torch.float64, device=dev)
            torch.cuda.synchronize()
            api.gemm_device(A32.data_ptr(), B32.data_ptr(), C32.data_ptr(), nn, nn, nn, opts)
            if api.sync_status() != 0:
                raise RuntimeError("kernel status non-zero")
            reps = 2
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(lib_stream)
            for _ in range(reps):
                api.gemm_device(A32.data_ptr(), B32.data_ptr(), C32.data_ptr(), nn, nn, nn, opts)
            f1.record(lib_stream)
            if api.sync_status() != 0:
                raise RuntimeError("kernel status non-zero")
            ms32 = f0.elapsed_time(f1) / reps
            one_gpu_sharded_shape = {"workload": "f64 GEMM 32768x32768x32768, exact tier, entries uniform[-1,1), one B200",
                                     "value": 2.0 * nn ** 3 / (ms32 * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms32,
                                     "steps": reps, "warmup": 1}
            del A32, B32, C32
        except (RuntimeError, MemoryError) as exc:  # reported, never fatal to the 8192^3 line
            one_gpu_sharded_shape = {"unavailable": str(exc).splitlines()[0][:200]}

    cpu = None
    if world == 1:
        cpu, _ = cpu_reference_run(n, 1024, 3, 1, "normal")

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": dict(workload_config(world), **({"b_panels": sg.panels, "b_panel_widths": [wd for _, wd in sg.cols], "transport": sg.transport, "rows_checked_against_one_gpu": verified} if sg else {})), "clocks": clocks,
        "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
    }
    if one_gpu_sharded_shape is not None:
        line["sharded_shape_on_one_gpu"] = one_gpu_sharded_shape
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def measure_int8_library_peak(torch, dev):
    """cuBLASLt int8 GEMM through torch._int_mm: the library's rate on this GPU, for context."""
    try:
        a = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device=dev).t().contiguous().t()
        for _ in range(3):
            torch._int_mm(a, b)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        return 10 * 2.0 * 8192 ** 3 / (e0.elapsed_time(e1) * 1e-3) / 1e12
    except Exception:  # noqa: BLE001 - context number only
        return None


def measure_fp64_library_peak(torch, dev):
    """torch.matmul f64 (cuBLAS DGEMM): the native FP64 rate the exact tier is compared with."""
    try:
        a = torch.randn((4096, 4096), dtype=torch.float64, device=dev)
        b = torch.randn((4096, 4096), dtype=torch.float64, device=dev)
        for _ in range(2):
            a @ b
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            a @ b
        e1.record()
        torch.cuda.synchronize()
        return 5 * 2.0 * 4096 ** 3 / (e0.elapsed_time(e1) * 1e-3) / 1e12
    except Exception:  # noqa: BLE001 - context number only
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
