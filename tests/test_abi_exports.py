"""The shared library loads without a GPU and exports every symbol include/*.h declares."""
import ctypes
import glob
import os
import re

import numpy as np
import pytest

import eshkol_b200 as eb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"\b(eshkol_[a-z0-9_]+)\s*\(", text):
            names.add(m.group(1))
        for m in re.finditer(r"extern\s+size_t\s+(\w+)\s*;", text):
            names.add(m.group(1))
    return sorted(names)


def test_headers_declare_the_reference_abi():
    names = declared_symbols()
    # the 32 functions + one global of inc/eshkol/backend/gpu/gpu_memory.h:90-474
    for required in ["eshkol_gpu_init", "eshkol_gpu_shutdown", "eshkol_gpu_get_backend",
                     "eshkol_gpu_backend_name", "eshkol_gpu_backend_available", "eshkol_gpu_supports_f64",
                     "eshkol_gpu_has_fp64", "eshkol_gpu_alloc", "eshkol_gpu_alloc_aligned", "eshkol_gpu_free",
                     "eshkol_gpu_wrap_host", "eshkol_gpu_sync", "eshkol_gpu_sync_async", "eshkol_gpu_wait",
                     "eshkol_gpu_matmul_f64", "eshkol_gpu_matmul_f32", "g_gpu_threshold",
                     "eshkol_gpu_set_threshold", "eshkol_gpu_get_threshold", "eshkol_gpu_should_use",
                     "eshkol_gpu_elementwise_f64", "eshkol_gpu_reduce_f64", "eshkol_gpu_reduce_axis_f64",
                     "eshkol_gpu_transpose_f64", "eshkol_gpu_softmax_f64", "eshkol_gpu_normalize_f64",
                     "eshkol_gpu_conv2d_backward_input_f64", "eshkol_gpu_conv2d_backward_kernel_f64",
                     "eshkol_gpu_batchnorm_backward_f64", "eshkol_gpu_layernorm_backward_f64",
                     "eshkol_matmul_dispatch", "eshkol_batch_matmul_dispatch"]:
        assert required in names, required


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(eb.library_path())
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_buffer_struct_layout_is_the_references():
    # inc/eshkol/backend/gpu/gpu_memory.h:60-68; mirrored by hand in lib/backend/vm_gpu_dispatch.h:60
    assert ctypes.sizeof(eb.EshkolGPUBuffer) == 48
    off = {f[0]: getattr(eb.EshkolGPUBuffer, f[0]).offset for f in eb.EshkolGPUBuffer._fields_}
    assert off == {"host_ptr": 0, "device_ptr": 8, "size_bytes": 16, "mem_type": 24, "backend": 28,
                   "flags": 32, "backend_data": 40}


def test_threshold_and_names_without_gpu():
    lib = eb.load_library()
    assert lib.eshkol_gpu_get_threshold() == 100000 or lib.eshkol_gpu_get_threshold() > 0
    old = lib.eshkol_gpu_get_threshold()
    lib.eshkol_gpu_set_threshold(12345)
    assert lib.eshkol_gpu_get_threshold() == 12345
    assert ctypes.c_size_t.in_dll(lib, "g_gpu_threshold").value == 12345
    lib.eshkol_gpu_set_threshold(old)
    assert lib.eshkol_gpu_backend_name(2) == b"NVIDIA CUDA"
    assert lib.eshkol_gpu_backend_name(0) == b"CPU (no GPU)"


def _choose(monkeypatch, env, shape=(2048, 2048, 2048)):
    for k in ["ESHKOL_B200_TIER", "ESHKOL_CUDA_F64_KERNEL", "ESHKOL_OZAKI_CUDA_T", "ESHKOL_MATMUL_ACCURACY",
              "ESHKOL_OZAKI_FAST", "ESHKOL_SF64_KERNEL", "ESHKOL_OZAKI_FAST_MODULI", "ESHKOL_OZAKI_NUM_MODULI"]:
        monkeypatch.delenv(k, raising=False)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    t, p = ctypes.c_int(), ctypes.c_int()
    eb.load_library().eshkol_b200_debug_choose_tier(*shape, ctypes.byref(t), ctypes.byref(p))
    return t.value, p.value


def test_tier_selection_follows_the_reference_switches(monkeypatch):
    assert _choose(monkeypatch, {}) == (eb.TIER_OZAKI2, 16)
    assert _choose(monkeypatch, {"ESHKOL_SF64_KERNEL": "ozaki", "ESHKOL_OZAKI_NUM_MODULI": "12"}) == (eb.TIER_OZAKI2, 12)
    # out of range moduli count: loud, default kept (lib/backend/gpu/gpu_memory.mm:1309-1314)
    assert _choose(monkeypatch, {"ESHKOL_OZAKI_NUM_MODULI": "17"}) == (eb.TIER_OZAKI2, 16)
    # lib/backend/gpu/gpu_memory_cuda.cpp:310-326, 462-464
    assert _choose(monkeypatch, {"ESHKOL_CUDA_F64_KERNEL": "ozaki-int8"}) == (eb.TIER_OZAKI1, 6)
    assert _choose(monkeypatch, {"ESHKOL_CUDA_F64_KERNEL": "ozaki-int8", "ESHKOL_OZAKI_CUDA_T": "4"}) == (eb.TIER_OZAKI1, 4)
    assert _choose(monkeypatch, {"ESHKOL_CUDA_F64_KERNEL": "ozaki-int8", "ESHKOL_OZAKI_CUDA_T": "99"}) == (eb.TIER_OZAKI1, 6)
    assert _choose(monkeypatch, {"ESHKOL_CUDA_F64_KERNEL": "ozaki-int8"}, (512, 512, 512)) == (eb.TIER_OZAKI2, 16)
    # accuracy budget: smallest T whose guaranteed error meets it (gpu_memory_cuda.cpp:485-487, 552-566)
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "fast"}) == (eb.TIER_OZAKI1, 1)
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "1e-9"}) == (eb.TIER_OZAKI1, 4)
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "exact"}) == (eb.TIER_OZAKI2, 16)
    # fast tier (gpu_memory.mm:1320-1337)
    assert _choose(monkeypatch, {"ESHKOL_OZAKI_FAST": "1"}) == (eb.TIER_OZAKI2_FAST, 11)
    assert _choose(monkeypatch, {"ESHKOL_SF64_KERNEL": "ozaki-fast", "ESHKOL_OZAKI_FAST_MODULI": "14"}) == (eb.TIER_OZAKI2_FAST, 14)
    assert _choose(monkeypatch, {"ESHKOL_OZAKI_FAST": "1", "ESHKOL_OZAKI_FAST_MODULI": "40"}) == (eb.TIER_OZAKI2_FAST, 16)
    assert _choose(monkeypatch, {"ESHKOL_B200_TIER": "dgemm"}) == (eb.TIER_DGEMM, 0)


def test_accuracy_budget_selector_consults_the_time_model(monkeypatch):
    """cuda_select_f64 (lib/backend/gpu/gpu_memory_cuda.cpp:552-575): the smallest T that meets the
    budget is taken only when the model predicts it 1.15 x faster than the full-precision kernel
    (here the Ozaki-II exact tier), only for shapes whose dimensions all reach 1024
    (cuda_ozaki_worthwhile, :462-464), and the model follows the best rate a kernel has shown."""
    lib = eb.load_library()
    ov, pk = ctypes.c_double(), ctypes.c_double()
    lib.eshkol_b200_debug_gemm_model(0, ctypes.byref(ov), ctypes.byref(pk))
    full = (ov.value, pk.value)
    lib.eshkol_b200_debug_gemm_model(5, ctypes.byref(ov), ctypes.byref(pk))
    t5 = (ov.value, pk.value)
    n = 4096
    work = 2.0 * n ** 3
    # T = 5 is slower than the exact tier on a B200: a 1e-11 budget stays exact, a 1e-9 budget takes T = 4
    assert (t5[0] + work / t5[1]) * 1.15 > full[0] + work / full[1]
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "1e-11"}, (n, n, n)) == (eb.TIER_OZAKI2, 16)
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "1e-9"}, (n, n, n)) == (eb.TIER_OZAKI1, 4)
    # budgets no slice tier guarantees, and the words for them, keep the exact tier
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "1e-15"}, (n, n, n)) == (eb.TIER_OZAKI2, 16)
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "full"}, (n, n, n)) == (eb.TIER_OZAKI2, 16)
    # a dimension below 1024: the slice tiers do not amortise their passes
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "fast"}, (512, n, n)) == (eb.TIER_OZAKI2, 16)
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "fast"}, (n, 1000, n)) == (eb.TIER_OZAKI2, 16)
    # K beyond the int32-exact bound of a slice product
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "fast"}, (2048, 140000, 2048)) == (eb.TIER_OZAKI2, 16)
    # calibration is a high-water mark: a slower measurement changes nothing, a faster one does
    lib.eshkol_b200_debug_gemm_calibrate(5, work, t5[0] + work / (t5[1] * 0.5))
    lib.eshkol_b200_debug_gemm_model(5, ctypes.byref(ov), ctypes.byref(pk))
    assert pk.value == t5[1]
    lib.eshkol_b200_debug_gemm_calibrate(5, work, t5[0] + work / (t5[1] * 3.0))
    lib.eshkol_b200_debug_gemm_model(5, ctypes.byref(ov), ctypes.byref(pk))
    assert abs(pk.value / (t5[1] * 3.0) - 1.0) < 1e-9
    assert _choose(monkeypatch, {"ESHKOL_MATMUL_ACCURACY": "1e-11"}, (n, n, n)) == (eb.TIER_OZAKI1, 5)
    # a measurement shorter than the fixed cost carries no rate
    lib.eshkol_b200_debug_gemm_calibrate(6, work, 1.0)
    lib.eshkol_b200_debug_gemm_model(6, ctypes.byref(ov), ctypes.byref(pk))
    assert pk.value < 1e6


def test_tensor_struct_layout_is_the_references():
    # lib/core/arena_memory.h:768-785: five 8-byte fields, 40 bytes, dtype appended at index 4
    from eshkol_b200.abi import EshkolTensor
    assert ctypes.sizeof(EshkolTensor) == 40
    off = {f[0]: getattr(EshkolTensor, f[0]).offset for f in EshkolTensor._fields_}
    assert off == {"dimensions": 0, "num_dimensions": 8, "elements": 16, "total_elements": 24, "dtype": 32}


def test_c_host_compiled_against_the_reference_headers_links():
    """tests/c_harness: a C program that includes the reference's own gpu_memory.h and
    vm_gpu_dispatch.h, built by oracle/Makefile (where the reference tree is present) and linked
    to this library; `link` takes the address of all 31 functions and checks the 48-byte buffer."""
    import subprocess
    exe = os.path.join(ROOT, "oracle", "_ref", "c_harness")
    if os.path.isdir("/root/reference"):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-s", "_ref/c_harness"], check=True,
                       capture_output=True)
    if not os.path.exists(exe):
        pytest.skip("the harness is built where the reference tree is present")
    r = subprocess.run([exe, "link"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "linked 31 functions" in r.stdout and "sizeof(EshkolGPUBuffer) = 48" in r.stdout


def test_inputs_stream_is_drand48():
    from eshkol_b200 import inputs
    libc = ctypes.CDLL(None)
    libc.drand48.restype = ctypes.c_double
    libc.srand48(12345)
    want = np.array([libc.drand48() for _ in range(4097)])
    got = inputs.lcg_states(12345, 4097).astype(np.float64) / float(1 << 48)
    assert np.array_equal(got, want)
    import torch
    st = inputs.lcg_states(12345, 4097, device="cpu").numpy().astype(np.uint64)
    assert np.array_equal(st, inputs.lcg_states(12345, 4097))
    u = inputs.uniform(1, (8, 8))
    assert u.min() >= -1.0 and u.max() < 1.0
    w = inputs.wide(2, (64, 64))
    assert np.abs(w).max() < 2.0 ** 20 and np.abs(w[w != 0]).min() < 2.0 ** -12
    f = inputs.full53(3, (4096,))
    assert (np.frombuffer(((f + 1.0) / 2.0 * 2.0 ** 53).astype(np.uint64).tobytes(), dtype=np.uint64) & np.uint64(15)).any()


def test_calls_fail_loudly_without_a_device():
    lib = eb.load_library()
    if lib.eshkol_gpu_init() == 1:
        pytest.skip("a GPU is present")
    a = np.ones((4, 4))
    buf = eb.EshkolGPUBuffer()
    assert lib.eshkol_gpu_matmul_f64(ctypes.byref(buf), ctypes.byref(buf), ctypes.byref(buf), 4, 4, 4) == -1
    assert lib.eshkol_b200_gemm_f64_device(a.ctypes.data, a.ctypes.data, a.ctypes.data, 4, 4, 4, None) == -1
    # the void dispatcher must not leave a plausible number behind
    c = eb.matmul_dispatch(a, a)
    assert np.isnan(c).all()
    # the other operators: -1 from the buffer level and from the device level, nothing computed
    out = np.full((4, 4), 7.0)
    hb = eb.EshkolGPUBuffer()
    hb.host_ptr = a.ctypes.data
    hb.size_bytes = a.nbytes
    ob = eb.EshkolGPUBuffer()
    ob.host_ptr = out.ctypes.data
    ob.size_bytes = out.nbytes
    dims = (ctypes.c_uint64 * 2)(4, 4)
    assert lib.eshkol_gpu_reduce_f64(ctypes.byref(hb), ctypes.byref(ob), 16, 0) == -1
    assert lib.eshkol_gpu_reduce_axis_f64(ctypes.byref(hb), ctypes.byref(ob), 2, dims, 0, 0) == -1
    assert lib.eshkol_gpu_transpose_f64(ctypes.byref(hb), ctypes.byref(ob), 4, 4) == -1
    assert lib.eshkol_gpu_softmax_f64(ctypes.byref(hb), ctypes.byref(ob), 4, 4) == -1
    assert lib.eshkol_gpu_normalize_f64(ctypes.byref(hb), ctypes.byref(ob), 4, 4, 1.0, 0.0, 1e-5) == -1
    assert lib.eshkol_gpu_batchnorm_backward_f64(*([ctypes.byref(hb)] * 5 + [ctypes.byref(ob)] * 3), 4, 4) == -1
    assert lib.eshkol_gpu_layernorm_backward_f64(*([ctypes.byref(hb)] * 5 + [ctypes.byref(ob)]), 4, 4) == -1
    assert lib.eshkol_b200_reduce_f64_device(a.ctypes.data, out.ctypes.data, 16, 0) == -1
    assert lib.eshkol_b200_softmax_f64_device(a.ctypes.data, out.ctypes.data, 4, 4) == -1
    assert lib.eshkol_b200_transpose_f64_device(a.ctypes.data, out.ctypes.data, 4, 4) == -1
    assert (out == 7.0).all()


def test_public_headers_are_plain_c(tmp_path):
    """Every header under include/ compiles as C99 on its own (the hosts are C programs)."""
    import glob
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    for h in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        src = tmp_path / (os.path.basename(h) + ".c")
        src.write_text(f'#include "{h}"\nint main(void) {{ return 0; }}\n')
        r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", str(src)],
                           capture_output=True, text=True)
        assert r.returncode == 0, h + "\n" + r.stderr
