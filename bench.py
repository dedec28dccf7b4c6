#!/usr/bin/env python
"""Benchmark of the f64 GEMM hot path (Ozaki-II exact tier).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N = 1: 8192^3, standard-normal operands, exact tier (the single-GPU configuration
the headline metric is quoted on).  N > 1 (launched under torch.distributed.run):
32768^3, uniform[-1,1) operands, rows of A sharded across the ranks, B distributed
from rank 0 and C gathered on every rank over NVLink, all inside the timed step.
One JSON line is printed by rank 0.  Outside the timed region the line's result is
compared with the CPU oracle (rows of the timed C, bit for bit); a run whose rows
differ prints no value.
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

# More hardware work queues than CUDA's default of 8: the sharded step keeps a dozen streams busy,
# and streams that share a queue wait for each other's event waits (a false dependency: a
# product then starts only when another panel's transfer has arrived).  Read when the CUDA
# context is created, so it has to be in the environment before torch initialises CUDA.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "f64-equivalent TFLOP/s, Ozaki-II exact GEMM"
UNIT = "TFLOP/s"
STAGES = ["scan_b", "split_b", "scan_a", "split_a", "products_mod256", "products_odd", "reconstruct"]

# guaranteed relative error of the slice tiers, T = 1..7 (lib/backend/gpu/gpu_memory_cuda.cpp:485-487)
OZAKI_TOL = {1: 1e-3, 2: 1e-5, 3: 1e-7, 4: 1e-9, 5: 1e-11, 6: 1e-13, 7: 1e-14}
# published worst-case error of the fast tier per moduli count (docs/breakdown/GPU_ACCELERATION.md:173-179)
FAST_TOL = {10: 2.2e-7, 11: 2.4e-8, 12: 4.0e-8, 14: 6e-11, 16: 6e-11}
# DRAM traffic of the two products kernels per launch, from the committed ncu capture at 4096^3
# (the profile summary of the odd-moduli kernel: 503.4 MB read + 230 MB written); the
# traffic is the operand planes re-read once per raster group plus the residue planes written,
# both proportional to M*N*K / (group rows) and M*N, so a launch at another shape scales as below
NCU_ODD_READ_4096, NCU_ODD_WRITE_4096 = 503.4e6, 230.0e6


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def parts_enabled():
    """ESHKOL_B200_BENCH_SKIP=tiers,conv,big,e2e,cpu,collectives leaves those sections out
    (development runs); the default run has every section."""
    skip = {s.strip() for s in os.environ.get("ESHKOL_B200_BENCH_SKIP", "").split(",") if s.strip()}
    return lambda name: name not in skip


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


def oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    return ol


# ------------------------------------------------------------------ reference arm
def cpu_reference_run(n_full: int, rows: int, steps: int, warmup: int, dist_name: str):
    """The reference's own CPU matmul (eshkol_matmul_f64, lib/backend/blas_backend.cpp:791)
    on a slab of `rows` rows of the n_full^3 product, on every host core this process may use."""
    cores = host_threads()
    # OpenBLAS and libgomp read their environment when they are loaded; a launcher such as
    # torch.distributed.run exports OMP_NUM_THREADS=1.  Set both before the first load and
    # again through the libraries' own setters afterwards, and report what they answer.
    os.environ["OPENBLAS_NUM_THREADS"] = str(cores)
    os.environ["OMP_NUM_THREADS"] = str(cores)
    ol = oracle()
    from eshkol_b200 import inputs
    gen = inputs.normal if dist_name == "normal" else inputs.uniform
    A = gen(1, (rows, n_full))
    B = gen(2, (n_full, n_full))
    kind, fn = "reference", None
    if ol.ref_lib("libref_matmul_blas.so") is not None:
        cores = ol.ref_blas_threads(cores)
        fn = lambda: ol.ref_matmul(A, B, blas=True)
        how = f"eshkol_matmul_f64 -> cblas_dgemm (OpenBLAS bundled in the image, openblas_get_num_threads = {cores})"
    elif ol.ref_lib("libref_matmul_simd.so") is not None:
        fn, cores = (lambda: ol.ref_matmul(A, B, blas=False)), 1
        how = "eshkol_matmul_f64 -> matmul_simd_avx (single thread by construction)"
    else:
        kind = "port"
        cores = ol.set_threads(cores)
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


def workload_config(n_gpus: int):
    if n_gpus == 1:
        return {"workload": "f64 GEMM 8192x8192x8192, exact (Ozaki-II, 16 moduli) tier, entries standard normal "
                            "(48-bit LCG + Box-Muller), single B200", "M": 8192, "K": 8192, "N": 8192,
                "l2": "operands (512 MiB each) exceed the 126 MB L2; no explicit flush"}
    return {"workload": "f64 GEMM 32768x32768x32768, exact tier, entries uniform[-1,1), rows of A sharded across "
                        f"{n_gpus} B200, B distributed from rank 0 and C gathered on every rank over NVLink inside the step",
            "M": 32768, "K": 32768, "N": 32768, "parallelism": f"row-shard x{n_gpus}",
            "l2": "operands exceed the 126 MB L2; no explicit flush"}


# ------------------------------------------------------------------- parity checks
def parity_rows(torch, A_rows_dev, B_dev, C_rows_dev, cols=None):
    """Rows of a timed result against the CPU oracle of the exact tier, bit for bit.  A_rows_dev:
    r x K rows of A; B_dev: K x N; C_rows_dev: the same r rows of C; cols: optional column
    sample (an index tensor) -- the oracle then multiplies those columns only."""
    import numpy as np
    ol = oracle()
    ol.set_threads(host_threads())
    A = A_rows_dev.cpu().numpy()
    if cols is None:
        B = B_dev.cpu().numpy()
        C = C_rows_dev.cpu().numpy()
    else:
        B = B_dev[:, cols].contiguous().cpu().numpy()
        C = C_rows_dev[:, cols].contiguous().cpu().numpy()
    t0 = time.perf_counter()
    want = ol.oz2_exact(A, B, 52)
    same = bool(np.array_equal(np.ascontiguousarray(C).view(np.uint64), want.view(np.uint64)))
    return same, time.perf_counter() - t0


def tier_block(torch, lib, api, eb, A, B, C_exact, n, lib_stream):
    """BASELINE config 3: every reduced tier at 8192^3 on the headline operands -- rate (timed on
    its own, outside the headline region) and error against two references: the exact tier's
    result (the reference's arithmetic, whose CRT accumulation itself rounds in a fraction of the
    cells) and the 16-moduli fast tier (integer CRT, nothing rounds before the final conversion:
    the closest thing to the true product the GPU holds at this size).  Errors are the maximum
    element-wise relative error with the denominator rule of the reference's probes
    (|ref| > 1e-9 ? |ref| : 1, tests/gpu/ozaki_correctness_test.esk:64-65) and the normwise
    Frobenius error (tests/gpu/cuda_ozaki_correctness_gate.sh:99-118); the documented bounds are
    normwise figures and are compared with the error against the fast-16 result."""
    out = []
    C = torch.empty((n, n), dtype=torch.float64, device=A.device)

    def errors(R):
        diff = (C - R).abs()
        denom = torch.where(R.abs() > 1e-9, R.abs(), torch.ones_like(R))
        return float((diff / denom).max()), float(torch.linalg.norm(diff) / torch.linalg.norm(R))

    def timed(run, reps=2):
        run()
        if api.sync_status() != 0:
            raise RuntimeError("kernel status non-zero")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(lib_stream)
        for _ in range(reps):
            run()
        e1.record(lib_stream)
        if api.sync_status() != 0:
            raise RuntimeError("kernel status non-zero")
        return e0.elapsed_time(e1) / reps

    plans = [(f"ozaki2-fast-{m}", eb.TIER_OZAKI2_FAST, m, FAST_TOL[m],
              "docs/breakdown/GPU_ACCELERATION.md:173-179 (worst case over the gate regimes)")
             for m in (16, 10, 11, 12, 14)]
    plans += [(f"ozaki1-T{t}", eb.TIER_OZAKI1, t, OZAKI_TOL[t], "OZAKI_TOL, gpu_memory_cuda.cpp:485-487")
              for t in range(1, 8)]
    C_best = None
    for name, tier, param, bound, src in plans:
        opts = api.make_opts(tier, param)
        ms = timed(lambda: api.gemm_device(A.data_ptr(), B.data_ptr(), C.data_ptr(), n, n, n, opts))
        if C_best is None:
            C_best = C.clone()
            mx, nw = errors(C_exact)
            out.append({"tier": "ozaki2-exact-16 (the headline)", "max_rel_err_vs_fast16": mx,
                        "normwise_err_vs_fast16": nw, "note": "the reference's exact-tier arithmetic measured "
                        "against the integer-CRT result; reproduced bit for bit (see parity)"})
        mx, nw = errors(C_exact)
        mxb, nwb = errors(C_best)
        out.append({"tier": name, "ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9, "max_rel_err_vs_exact": mx,
                    "normwise_err_vs_exact": nw, "max_rel_err_vs_fast16": mxb, "normwise_err_vs_fast16": nwb,
                    "documented_bound": bound, "bound_source": src, "within_bound": bool(nwb <= bound)})

    def f16():
        if lib.eshkol_b200_gemm_f16_device(A.data_ptr(), B.data_ptr(), C.data_ptr(), 1, n, n, n) != 0:
            raise RuntimeError("gemm_f16 failed")
    ms = timed(f16)
    mx, nw = errors(C_exact)
    mxb, nwb = errors(C_best)
    out.append({"tier": "f16 dtype path (f64 storage, f16 operands, f32 accumulation)", "ms": ms,
                "tflops": 2.0 * n ** 3 / ms / 1e9, "max_rel_err_vs_exact": mx, "normwise_err_vs_exact": nw,
                "max_rel_err_vs_fast16": mxb, "normwise_err_vs_fast16": nwb,
                "documented_bound": None, "bound_source": "none documented by the reference (parity unpinned)",
                "within_bound": None})
    return out


def conv_c4_block(torch, lib, api, eb, dev, lib_stream, with_cpu):
    """BASELINE config 4: conv2d NCHW batch 32, 64 -> 128 channels, 56 x 56, 3 x 3, stride 1,
    pad 1, inputs and weights normal(0, 0.1), fused ReLU, exact tier; device-resident tensors."""
    from eshkol_b200 import inputs
    b, ic, H, W, oc, kh, kw, stride, pad = 32, 64, 56, 56, 128, 3, 3, 1, 1
    x = inputs.normal(1, (b, ic, H, W), device=dev, scale=0.1)
    w = inputs.normal(2, (oc, ic, kh, kw), device=dev, scale=0.1)
    y = torch.empty((b, oc, H, W), dtype=torch.float64, device=dev)
    torch.cuda.synchronize()
    opts = api.make_opts(eb.TIER_OZAKI2, 16, activation=1)

    def run():
        api.conv2d_device(x.data_ptr(), (b, ic, H, W), w.data_ptr(), (oc, ic, kh, kw), stride, pad, y.data_ptr(), opts)
    for _ in range(2):
        run()
    if api.sync_status() != 0:
        raise RuntimeError("kernel status non-zero")
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(lib_stream)
    for _ in range(reps):
        run()
    e1.record(lib_stream)
    if api.sync_status() != 0:
        raise RuntimeError("kernel status non-zero")
    ms = e0.elapsed_time(e1) / reps
    flop = 2.0 * oc * (ic * kh * kw) * (b * H * W)
    moved = (x.numel() + w.numel() + y.numel()) * 8
    out = {"workload": "conv2d f64 NCHW 32x64x56x56 * 128x64x3x3, stride 1, pad 1, ReLU fused, exact tier "
                       "(GEMM 128 x 576 x 100352)", "ms": ms, "tflops": flop / ms / 1e9,
           "algorithmic_gb": moved / 1e9, "gb_per_s_algorithmic": moved / ms / 1e6}
    if with_cpu:
        # the reference's eshkol_conv2d_kernel (lib/backend/tensor_conv_kernel.h:66-105) is one
        # thread by construction; timed on 2 of the 32 images
        ol = oracle()
        sub = 2
        xs = x[:sub].cpu().numpy()
        ws = w.cpu().numpy()
        t0 = time.perf_counter()
        ref = ol.ref_conv2d(xs, ws, stride, pad)
        dt = time.perf_counter() - t0
        if ref is not None:
            import numpy as np
            got = y[:sub].cpu().numpy()
            relu = np.maximum(ref, 0.0)
            out["cpu_baseline"] = {"value": flop * sub / b / dt / 1e12, "unit": UNIT, "cores": 1, "kind": "reference",
                                   "sample": f"eshkol_conv2d_kernel on {sub} of the {b} images, one pass"}
            out["max_abs_diff_vs_reference_kernel"] = float(np.max(np.abs(got - relu)))
    return out


# ----------------------------------------------------------------------- our arm
def run_b200(args):
    import numpy as np
    import torch
    import eshkol_b200 as eb
    from eshkol_b200 import api, inputs

    want = parts_enabled()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    comm_sms = int(os.environ.get("ESHKOL_B200_COMM_SMS", "0"))  # measured: capping the collectives' CTAs costs more than it frees
    if world > 1:
        import datetime
        import torch.distributed as dist_mod
        dist = dist_mod
        if comm_sms > 0:
            # the collectives run on the SMs the products kernels leave free (see ShardedGemm)
            os.environ.setdefault("NCCL_MAX_CTAS", str(comm_sms))
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=900))
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
        # column panels of B overlap the distribution and the gather with the products
        panels = int(os.environ.get("ESHKOL_B200_PANELS", "4"))
        transport = os.environ.get("ESHKOL_B200_TRANSPORT", "copy_engine")
        # every rank splits 1/N of each panel's columns and the residue planes are exchanged,
        # instead of every rank splitting all of B
        share = os.environ.get("ESHKOL_B200_SHARE_SPLIT", "1") == "1"
        # narrow first and last panels shorten the two transfers nothing hides
        taper = os.environ.get("ESHKOL_B200_TAPER", "gentle" if share else "geometric")
        # the schedule itself runs in C (include/eshkol_b200_multi.h); ESHKOL_B200_DRIVER=python
        # selects the same schedule written over torch.distributed, which also has the variants
        if os.environ.get("ESHKOL_B200_DRIVER", "c") == "c" and share and transport == "copy_engine":
            from eshkol_b200.sharded import CShardedGemm
            sg = CShardedGemm(n, n, n, dev, rank=rank, world=world)
        else:
            sg = ShardedGemm(n, n, n, dev, tier=eb.TIER_OZAKI2, param=16, panels=panels, comm_sms=comm_sms,
                             transport=transport, taper=taper, share_split=share, b_in_place=share)
        rows = sg.rows
        A = inputs.uniform(1, (rows, n), device=dev, start=sg.row0 * n)
        B = None
        if rank == 0:
            # B lives in the buffer the peers have opened, so the source GPU packs nothing
            B = sg.source_buffer() if sg.b_in_place and sg.split_shared else None
            if B is not None:
                B.copy_(inputs.uniform(2, (n, n), device=dev))
            else:
                B = inputs.uniform(2, (n, n), device=dev)
        C_local = None
    torch.cuda.synchronize()

    def step(g=None):
        if world == 1:
            api.gemm_device(A.data_ptr(), B.data_ptr(), C_local.data_ptr(), n, n, n, opts)
        else:
            (g or sg).step(A, B)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if api.sync_status() != 0:
            raise RuntimeError("kernel status non-zero")

    def timed_steps(g=None):
        """K steps bracketed by a barrier and a device synchronisation on both sides; CUDA events on
        the stream the steps are enqueued on; the maximum over the ranks."""
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        barrier()
        if world == 1:
            ev0.record(lib_stream)
            for _ in range(args.steps):
                step()
            ev1.record(lib_stream)
            barrier()
            return ev0.elapsed_time(ev1)
        # the step mixes the library stream, copy streams and (collectives transport) torch's
        # stream; its last action is a synchronisation of torch's stream behind all of them
        ev0.record(torch.cuda.current_stream())
        for _ in range(args.steps):
            step(g)
        torch.cuda.current_stream().synchronize()
        ev1.record(torch.cuda.current_stream())
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

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
        # every rank must run the same number of steps: a fixed count (a step of the sharded
        # configuration takes 0.07 - 0.26 s)
        for _ in range(8):
            step()
            soak_steps += 1
    barrier()
    # stage events are recorded inside the timed steps themselves and summed afterwards
    lib.eshkol_b200_set_phase_timing(1)
    launches0 = api.launch_count()
    ms_total = timed_steps()
    launches = api.launch_count() - launches0
    ph = (ctypes.c_float * 7)()
    cnt = (ctypes.c_int * 3)()
    got = lib.eshkol_b200_get_phase_totals(ph, cnt)
    lib.eshkol_b200_set_phase_timing(0)
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = f"{soak_steps} identical untimed steps directly before + the {args.steps} timed steps"
    ms_step = ms_total / args.steps
    value = 2.0 * n * n * n / (ms_step * 1e-3) / 1e12
    phases = [float(x) / args.steps for x in ph] if got == 0 and cnt[2] > 0 else None  # per step, this rank

    # ---- a second transport's number for the sharded configuration (NCCL collectives) ----
    collectives = None
    if sg is not None and sg.transport != "collectives" and want("collectives"):
        from eshkol_b200.sharded import ShardedGemm
        sg_c = ShardedGemm(n, n, n, dev, tier=eb.TIER_OZAKI2, param=16, panels=4, transport="collectives")
        for _ in range(2):
            step(sg_c)
        ms_c = timed_steps(sg_c) / args.steps
        collectives = {"transport": "collectives (ncclBroadcast of B panels, ncclAllGather of C blocks)",
                       "ms_per_step": ms_c, "value": 2.0 * n ** 3 / (ms_c * 1e-3) / 1e12, "unit": UNIT, "b_panels": 4}
        sg_c.close()
        del sg_c
        torch.cuda.empty_cache()

    # ---- parity of the timed result (outside the timed region) ----
    parity = None
    if world == 1:
        # rows of the C the timed steps wrote, against the CPU oracle
        g = torch.Generator().manual_seed(5)
        pick = torch.randperm(n, generator=g)[:16].sort().values.to(dev)
        same, secs = parity_rows(torch, A[pick], B, C_local[pick])
        parity = {"rows": int(pick.numel()), "cols": n, "bitwise": same, "against": "CPU oracle of the exact tier",
                  "oracle_seconds": secs}
    else:
        # every rank's C must be the same matrix: a wrapping 64-bit sum of its bit patterns
        cks = sg.C.view(torch.int64).sum().reshape(1)
        allc = [torch.zeros_like(cks) for _ in range(world)]
        dist.all_gather(allc, cks)
        cross = all(int(c.item()) == int(allc[0].item()) for c in allc)
        if rank == 0:
            # rows taken from every rank's block x sampled columns, against the CPU oracle
            per = max(8, 64 // world)
            g = torch.Generator().manual_seed(5)
            pick = torch.cat([r0 + torch.randperm(rr, generator=g)[:per].sort().values for r0, rr in sg.parts]).to(dev)
            cols = torch.randperm(n, generator=g)[:512].sort().values.to(dev)
            A_rows = torch.cat([inputs.uniform(1, (1, n), device=dev, start=int(i) * n) for i in pick.tolist()])
            same, secs = parity_rows(torch, A_rows, B, sg.C[pick], cols)
            parity = {"rows": int(pick.numel()), "rows_per_rank_block": per, "cols": int(cols.numel()), "bitwise": same,
                      "against": "CPU oracle of the exact tier", "oracle_seconds": secs,
                      "identical_on_every_rank": cross}
            if not cross:
                parity["bitwise"] = False
            del A_rows

    # ---- the sharded shape on one GPU, the denominator of the parallel efficiency ----
    one_gpu = None
    if want("big"):
        if world > 1:
            dist.barrier()  # rank 0 alone multiplies 32768^3 below; the others wait at the next barrier
        if rank == 0:
            try:
                if world == 1:
                    A32 = inputs.uniform(1, (32768, 32768), device=dev)
                    B32 = inputs.uniform(2, (32768, 32768), device=dev)
                    C32 = torch.empty((32768, 32768), dtype=torch.float64, device=dev)
                else:
                    A32 = inputs.uniform(1, (n, n), device=dev)
                    B32, C32 = B, torch.empty((n, n), dtype=torch.float64, device=dev)
                nn = 32768
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
                one_gpu = {"workload": "f64 GEMM 32768x32768x32768, exact tier, entries uniform[-1,1), one B200",
                           "value": 2.0 * nn ** 3 / (ms32 * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms32,
                           "steps": reps, "warmup": 1}
                if world > 1:
                    one_gpu["same_bits_as_the_sharded_result"] = bool(
                        torch.equal(C32.view(torch.int64), sg.C.view(torch.int64)))
                del A32, B32, C32
                torch.cuda.empty_cache()
            except (RuntimeError, MemoryError) as exc:  # reported, never fatal to the headline line
                one_gpu = {"unavailable": str(exc).splitlines()[0][:200]}
        if world > 1:
            dist.barrier()

    if rank != 0:
        if sg is not None:
            sg.close()
        dist.destroy_process_group()
        return

    peaks = measured_peaks()
    roofline = None
    if phases:
        # products of the odd moduli: 15 int8 GEMMs over this rank's rows
        t_odd = phases[5] * 1e-3
        ops = 15 * 2.0 * rows * n * n
        achieved = ops / t_odd / 1e12
        int8_peak = measure_int8_library_peak(torch, dev)
        peak2 = 2.0 * peaks["bf16_tflops_sustained"]
        peak = int8_peak or peak2
        scale = (rows / 4096.0) * (n / 4096.0) * (n / 4096.0)
        roofline = {
            "kernel": "modgemm_kernel<256, odd moduli> (tcgen05 int8 -> int32, 15 planes)",
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "traffic": (NCU_ODD_READ_4096 + NCU_ODD_WRITE_4096) * scale if world == 1 else None,
            "traffic_source": "ncu dram__bytes_read + dram__bytes_write of the kernel at 4096^3 "
                              "(committed profile summary), scaled by M*K*N: the planes are re-read once per group of m-tiles",
            "peak_source": ("cuBLASLt int8 GEMM 8192^3 (torch._int_mm) timed live in this run after the timed region"
                            if int8_peak else f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']})"),
            "peak_2x_bf16_sustained": peak2, "frac_of_2x_bf16_sustained": achieved / peak2,
            "timed": f"CUDA events on the library stream inside the {args.steps} timed steps, summed per stage",
            "phases_ms": dict(zip(STAGES, phases)),
            "phase_calls": {"prepare_b": int(cnt[0]), "prepare_a": int(cnt[1]), "multiply": int(cnt[2])},
        }
        if world == 1:
            roofline["unaccounted_ms"] = ms_step - sum(phases)
        # the memory-side stages against the measured copy bandwidth: algorithmic bytes per
        # element are 8 read + 15 (odd planes) + 1024/1008 (modulus-256 plane) + 0.25 (flag
        # bit-planes) written for a split, 15 + 2 + 0.125 read + 8 written for the reconstruction
        kn = float(n) * n
        mk = float(rows) * n
        mn = float(rows) * n
        split_bytes = 8.0 + 15.0 + 1024.0 / 1008.0 + 0.25
        stages = [("scan_cols (B)", 8.0 * kn, phases[0]), ("split_b", split_bytes * kn, phases[1]),
                  ("scan_rows (A)", 8.0 * mk, phases[2]), ("split_a", split_bytes * mk, phases[3]),
                  ("crt (reconstruction)", (17.125 + 8.0) * mn, phases[6])]
        roofline["hbm_stages"] = [
            {"kernel": name, "bound": "hbm", "achieved": b / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
             "unit": "GB/s", "frac": b / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "ms": ms}
            for name, b, ms in stages if ms > 0]
        fp64 = measure_fp64_library_peak(torch, dev)
        if fp64:
            roofline["native_fp64_gemm_tflops_live"] = fp64
            roofline["value_vs_native_fp64"] = value / world / fp64

    tiers = None
    if world == 1 and want("tiers"):
        tiers = tier_block(torch, lib, api, eb, A, B, C_local, n, lib_stream)

    # end to end through the reference-facing dispatcher, host buffers
    e2e = None
    e2e_pageable = None
    e2e_reused_b = None
    if world == 1 and want("e2e"):
        lib.eshkol_gpu_init()

        def dispatch_rate(hA, hB, hC, reps):
            for _ in range(2):
                lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
            t0 = time.perf_counter()
            for _ in range(reps):
                lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
            return (time.perf_counter() - t0) / reps
        e2e_steps = max(2, min(args.steps, 5))
        hA = torch.empty((n, n), dtype=torch.float64).pin_memory()
        hB = torch.empty((n, n), dtype=torch.float64).pin_memory()
        hC = torch.empty((n, n), dtype=torch.float64).pin_memory()
        hA.copy_(A)
        hB.copy_(B)
        torch.cuda.synchronize()
        dt = dispatch_rate(hA, hB, hC, e2e_steps)
        e2e = {"value": 2.0 * n * n * n / dt / 1e12, "unit": UNIT, "h2d_bytes_per_step": 2 * n * n * 8,
               "d2h_bytes_per_step": n * n * 8, "ms_per_step": dt * 1e3,
               "api": "eshkol_matmul_dispatch(host A, host B, host C), pinned host memory",
               "same_bits_as_the_device_result": bool(torch.equal(hC.view(torch.int64), C_local.cpu().view(torch.int64)))}
        # the reference's callers pass arena memory, which is pageable (llvm_codegen.cpp:32194-32218)
        pA, pB, pC = hA.clone(), hB.clone(), torch.empty((n, n), dtype=torch.float64)
        assert not pA.is_pinned()
        dt = dispatch_rate(pA, pB, pC, e2e_steps)
        e2e_pageable = {"value": 2.0 * n * n * n / dt / 1e12, "unit": UNIT, "ms_per_step": dt * 1e3,
                        "api": "eshkol_matmul_dispatch(host A, host B, host C), pageable host memory",
                        "same_bits_as_the_device_result": bool(torch.equal(pC.view(torch.int64), C_local.cpu().view(torch.int64)))}
        # operands that stay on the device between calls (the dispatcher's residency cache): B is
        # found on the device and is still the prepared operand, so nothing of it is uploaded or
        # split again; A is declared changed before every call, as fresh activations would be
        lib.eshkol_gpu_set_residency(1, 32768)
        try:
            for _ in range(3):
                lib.eshkol_gpu_invalidate(hA.data_ptr(), 0)
                lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
            moved0 = (ctypes.c_uint64(), ctypes.c_uint64())
            lib.eshkol_b200_transfer_bytes(ctypes.byref(moved0[0]), ctypes.byref(moved0[1]))
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                lib.eshkol_gpu_invalidate(hA.data_ptr(), 0)
                lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
            dt = (time.perf_counter() - t0) / e2e_steps
            moved1 = (ctypes.c_uint64(), ctypes.c_uint64())
            lib.eshkol_b200_transfer_bytes(ctypes.byref(moved1[0]), ctypes.byref(moved1[1]))
            e2e_reused_b = {"value": 2.0 * n * n * n / dt / 1e12, "unit": UNIT, "ms_per_step": dt * 1e3,
                            "h2d_bytes_per_step": (moved1[0].value - moved0[0].value) // e2e_steps,
                            "d2h_bytes_per_step": (moved1[1].value - moved0[1].value) // e2e_steps,
                            "api": "eshkol_matmul_dispatch with ESHKOL_B200_RESIDENCY=1, pinned host memory: B resident and "
                                   "prepared, A invalidated (uploaded) every call, C downloaded every call",
                            "same_bits_as_the_device_result": bool(torch.equal(hC.view(torch.int64), C_local.cpu().view(torch.int64)))}
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                lib.eshkol_matmul_dispatch(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), n, n, n, 0)
            dt = (time.perf_counter() - t0) / e2e_steps
            e2e_reused_b["both_operands_resident"] = {"value": 2.0 * n * n * n / dt / 1e12, "ms_per_step": dt * 1e3}
        finally:
            lib.eshkol_gpu_set_residency(0, 0)
        del hA, hB, hC, pA, pB, pC
    elif world > 1:
        e2e = {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "sharded configuration is defined on device-resident operands; see the 1-GPU line for PCIe"}

    conv = None
    if world == 1 and want("conv"):
        conv = conv_c4_block(torch, lib, api, eb, dev, lib_stream, want("cpu"))

    cpu = None
    if world == 1 and want("cpu"):
        cpu, _ = cpu_reference_run(n, 1024, 3, 1, "normal")

    config = workload_config(world)
    if sg is not None:
        config.update({"b_panels": sg.panels, "b_panel_widths": [wd for _, wd in sg.cols], "transport": sg.transport,
                       "b_prepared_once": getattr(sg, "split_shared", False)})
    line = {
        "metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": config, "clocks": clocks,
        "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu, "parity": parity,
    }
    if parity is not None and parity["bitwise"]:
        line["value"] = value
    else:
        line["value"] = None
        line["invalid"] = "the timed result differs from the oracle: no value is reported"
        if e2e is not None:
            e2e["value"] = None
    if e2e_pageable is not None:
        line["e2e_pageable"] = e2e_pageable
    if e2e_reused_b is not None:
        line["e2e_reused_b"] = e2e_reused_b
    if tiers is not None:
        line["tiers"] = tiers
    if conv is not None:
        line["conv_c4"] = conv
    if collectives is not None:
        line["collectives_transport"] = collectives
    if one_gpu is not None:
        if world == 1:
            line["sharded_shape_on_one_gpu"] = one_gpu
        else:
            line["one_gpu_same_shape"] = one_gpu
            if "value" in one_gpu:
                line["one_gpu_same_shape_tflops"] = one_gpu["value"]
                line["efficiency_vs_one_gpu_same_shape"] = value / (world * one_gpu["value"])
    print(json.dumps(line), flush=True)
    if sg is not None:
        sg.close()
    if dist is not None:
        dist.destroy_process_group()


def measure_int8_library_peak(torch, dev):
    """cuBLASLt int8 GEMM through torch._int_mm: the library's rate on this GPU in this run."""
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
