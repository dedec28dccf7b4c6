"""ctypes view of libeshkol_gpu_b200.so.

Struct layouts restate include/eshkol_gpu_memory_b200.h and
include/eshkol_b200_ext.h; the reference's own layout is
inc/eshkol/backend/gpu/gpu_memory.h:60-68 (EshkolGPUBuffer, 48 bytes on LP64).
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(HERE, "libeshkol_gpu_b200.so")

TIER_OZAKI2 = 0
TIER_OZAKI1 = 1
TIER_OZAKI2_FAST = 2
TIER_DGEMM = 3

c_double_p = ctypes.POINTER(ctypes.c_double)


class EshkolGPUBuffer(ctypes.Structure):
    _fields_ = [
        ("host_ptr", ctypes.c_void_p),
        ("device_ptr", ctypes.c_void_p),
        ("size_bytes", ctypes.c_size_t),
        ("mem_type", ctypes.c_int),
        ("backend", ctypes.c_int),
        ("flags", ctypes.c_uint32),
        ("backend_data", ctypes.c_void_p),
    ]


class EshkolTensor(ctypes.Structure):
    """eshkol_tensor_t (lib/core/arena_memory.h:768-780): 40 bytes, elements are doubles stored
    as int64 bit patterns."""
    _fields_ = [
        ("dimensions", ctypes.POINTER(ctypes.c_uint64)),
        ("num_dimensions", ctypes.c_uint64),
        ("elements", ctypes.POINTER(ctypes.c_int64)),
        ("total_elements", ctypes.c_uint64),
        ("dtype", ctypes.c_uint64),
    ]


class GemmOpts(ctypes.Structure):
    _fields_ = [
        ("tier", ctypes.c_int32),
        ("param", ctypes.c_int32),
        ("activation", ctypes.c_int32),
        ("bias_mode", ctypes.c_int32),
        ("bias", ctypes.c_void_p),
        ("pixels_per_image", ctypes.c_int64),
        ("use_simt_products", ctypes.c_int32),
        ("gemm_tile_n", ctypes.c_int32),
        ("ldc", ctypes.c_int64),
        ("trans_a", ctypes.c_int32),
        ("trans_b", ctypes.c_int32),
    ]


_lib = None


def library_path() -> str:
    return _LIB_PATH


def load_library() -> ctypes.CDLL:
    """Load the built library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is not built; run `python -m eshkol_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for this path."
        )
    lib = ctypes.CDLL(_LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    u64, i64, i32, vp = ctypes.c_uint64, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p
    bufp = ctypes.POINTER(EshkolGPUBuffer)
    optp = ctypes.POINTER(GemmOpts)

    def sig(name, res, args):
        f = getattr(lib, name)
        f.restype = res
        f.argtypes = args

    sig("eshkol_gpu_init", ctypes.c_int, [])
    sig("eshkol_gpu_shutdown", None, [])
    sig("eshkol_gpu_get_backend", ctypes.c_int, [])
    sig("eshkol_gpu_backend_name", ctypes.c_char_p, [ctypes.c_int])
    sig("eshkol_gpu_backend_available", ctypes.c_int, [ctypes.c_int])
    sig("eshkol_gpu_supports_f64", ctypes.c_int, [])
    sig("eshkol_gpu_has_fp64", ctypes.c_int, [])
    sig("eshkol_gpu_alloc", ctypes.c_int, [ctypes.c_size_t, ctypes.c_int, bufp])
    sig("eshkol_gpu_alloc_aligned", ctypes.c_int, [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, bufp])
    sig("eshkol_gpu_free", None, [bufp])
    sig("eshkol_gpu_wrap_host", ctypes.c_int, [vp, ctypes.c_size_t, bufp])
    sig("eshkol_gpu_sync", ctypes.c_int, [bufp, ctypes.c_int])
    sig("eshkol_gpu_sync_async", ctypes.c_int, [bufp, ctypes.c_int, vp])
    sig("eshkol_gpu_wait", None, [bufp])
    sig("eshkol_gpu_matmul_f64", ctypes.c_int, [bufp, bufp, bufp, u64, u64, u64])
    sig("eshkol_gpu_matmul_f32", ctypes.c_int, [bufp, bufp, bufp, u64, u64, u64])
    sig("eshkol_gpu_set_threshold", None, [ctypes.c_size_t])
    sig("eshkol_gpu_get_threshold", ctypes.c_size_t, [])
    sig("eshkol_gpu_should_use", ctypes.c_int, [ctypes.c_size_t])
    sig("eshkol_gpu_elementwise_f64", ctypes.c_int, [bufp, bufp, bufp, u64, ctypes.c_int])
    sig("eshkol_gpu_reduce_f64", ctypes.c_int, [bufp, bufp, u64, ctypes.c_int])
    sig("eshkol_gpu_reduce_axis_f64", ctypes.c_int, [bufp, bufp, u64, ctypes.POINTER(u64), u64, ctypes.c_int])
    sig("eshkol_gpu_transpose_f64", ctypes.c_int, [bufp, bufp, u64, u64])
    sig("eshkol_gpu_softmax_f64", ctypes.c_int, [bufp, bufp, u64, u64])
    sig("eshkol_gpu_normalize_f64", ctypes.c_int, [bufp, bufp, u64, u64, ctypes.c_double, ctypes.c_double, ctypes.c_double])
    sig("eshkol_gpu_batchnorm_backward_f64", ctypes.c_int, [bufp] * 8 + [u64, u64])
    sig("eshkol_gpu_layernorm_backward_f64", ctypes.c_int, [bufp] * 6 + [u64, u64])
    sig("eshkol_matmul_dispatch", None, [vp, vp, vp, u64, u64, u64, i32])
    sig("eshkol_batch_matmul_dispatch", None, [vp, vp, vp, i64, i64, i64, i64, i32])
    sig("eshkol_gpu_conv2d_f64", ctypes.c_int, [vp, i64, i64, i64, i64, vp, i64, i64, i64, i64, i64, vp, i32])
    sig("eshkol_gpu_matmul_backward_f64", ctypes.c_int, [vp, vp, vp, vp, vp, u64, u64, u64])
    sig("eshkol_b200_init", ctypes.c_int, [ctypes.c_int])
    sig("eshkol_b200_shutdown", None, [])
    sig("eshkol_b200_stream", vp, [])
    sig("eshkol_b200_gemm_f64_device", ctypes.c_int, [vp, vp, vp, u64, u64, u64, optp])
    sig("eshkol_b200_gemm_f64_static_scratch", ctypes.c_int, [vp, vp, vp, u64, u64, u64])
    sig("eshkol_b200_matmul_f64_host", ctypes.c_int, [vp, vp, vp, u64, u64, u64, optp])
    sig("eshkol_b200_feed_forward_f64_device", ctypes.c_int, [vp, vp, vp, vp, vp, vp, u64, u64, u64, optp])
    sig("eshkol_b200_conv2d_backward_kernel_f64_device", ctypes.c_int, [vp, vp, vp] + [u64] * 11 + [optp])
    sig("eshkol_b200_conv2d_backward_input_f64_device", ctypes.c_int, [vp, vp, vp] + [u64] * 11 + [optp])
    sig("eshkol_b200_gemm_f16_device", ctypes.c_int, [vp, vp, vp, u64, u64, u64, u64])
    sig("eshkol_b200_gemm_f32_device", ctypes.c_int, [vp, vp, vp, u64, u64, u64])
    sig("eshkol_b200_matmul_backward_f64_host", ctypes.c_int, [vp, vp, vp, vp, vp, u64, u64, u64, optp, optp])
    sig("eshkol_b200_prepare_b_f64_device", ctypes.c_int, [vp, u64, u64])
    sig("eshkol_b200_gemm_prepared_f64_device", ctypes.c_int, [vp, vp, u64, optp])
    sig("eshkol_b200_prepare_a_f64_device", ctypes.c_int, [vp, u64, u64, u64])
    sig("eshkol_b200_prepared_b_bytes", u64, [u64, u64])
    sig("eshkol_b200_prepare_b_columns_f64_device", ctypes.c_int, [vp, u64, u64, u64, u64, u64, vp])
    sig("eshkol_b200_prepared_b_regions", ctypes.c_int, [u64, u64, u64, u64, ctypes.POINTER(u64)])
    sig("eshkol_b200_adopt_prepared_b", ctypes.c_int, [vp, u64, u64])
    sig("eshkol_b200_multiply_prepared_f64_device", ctypes.c_int, [vp, optp])
    sig("eshkol_b200_conv2d_f64_device", ctypes.c_int, [vp, i64, i64, i64, i64, vp, i64, i64, i64, i64, i64, vp, optp])
    sig("eshkol_b200_mem_alloc", ctypes.c_int, [ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(vp)])
    sig("eshkol_b200_mem_free", None, [ctypes.c_int, vp])
    sig("eshkol_b200_copy_h2d", ctypes.c_int, [vp, vp, ctypes.c_size_t])
    sig("eshkol_b200_copy_d2h", ctypes.c_int, [vp, vp, ctypes.c_size_t])
    sig("eshkol_b200_elementwise_f64_device", ctypes.c_int, [vp, vp, vp, u64, ctypes.c_int])
    sig("eshkol_b200_reduce_f64_device", ctypes.c_int, [vp, vp, u64, ctypes.c_int])
    sig("eshkol_b200_reduce_axis_f64_device", ctypes.c_int, [vp, vp, u64, u64, u64, ctypes.c_int])
    sig("eshkol_b200_transpose_f64_device", ctypes.c_int, [vp, vp, u64, u64])
    sig("eshkol_b200_softmax_f64_device", ctypes.c_int, [vp, vp, u64, u64])
    sig("eshkol_b200_normalize_f64_device", ctypes.c_int, [vp, vp, u64, u64, ctypes.c_double, ctypes.c_double, ctypes.c_double])
    sig("eshkol_b200_batchnorm_backward_f64_device", ctypes.c_int, [vp] * 8 + [u64, u64])
    sig("eshkol_b200_layernorm_backward_f64_device", ctypes.c_int, [vp] * 6 + [u64, u64])
    sig("eshkol_b200_sync_status", ctypes.c_int, [])
    sig("eshkol_b200_set_pair_gemm", None, [ctypes.c_int])
    sig("eshkol_b200_set_sm_limit", None, [ctypes.c_int])
    sig("eshkol_b200_enable_peer_access", ctypes.c_int, [ctypes.c_int])
    sig("eshkol_b200_copy_async", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p])
    hp = ctypes.c_char_p
    sig("eshkol_b200_ipc_export_mem", ctypes.c_int, [vp, hp])
    sig("eshkol_b200_ipc_import_mem", ctypes.c_int, [hp, ctypes.POINTER(vp)])
    sig("eshkol_b200_ipc_close_mem", ctypes.c_int, [vp])
    sig("eshkol_b200_ipc_event_create", ctypes.c_int, [ctypes.POINTER(vp), hp])
    sig("eshkol_b200_ipc_event_import", ctypes.c_int, [hp, ctypes.POINTER(vp)])
    sig("eshkol_b200_event_record", ctypes.c_int, [vp, vp])
    sig("eshkol_b200_event_wait", ctypes.c_int, [vp, vp])
    sig("eshkol_b200_event_destroy", ctypes.c_int, [vp])
    sig("eshkol_b200_copy2d_async", ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t,
                                                   ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p])
    sig("eshkol_b200_set_row_bands", None, [ctypes.c_longlong])
    sig("eshkol_b200_set_phase_timing", None, [ctypes.c_int])
    sig("eshkol_b200_get_phase_times", ctypes.c_int, [ctypes.POINTER(ctypes.c_float), ctypes.c_int])
    sig("eshkol_b200_get_phase_totals", ctypes.c_int, [ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int)])
    sig("eshkol_b200_launch_count", u64, [])
    sig("eshkol_b200_workspace_bytes", u64, [])
    sig("eshkol_b200_matmul_f64_host_resident", ctypes.c_int, [vp, vp, vp, u64, u64, u64, vp, ctypes.c_int, vp, ctypes.c_int,
                                                                vp, ctypes.POINTER(u64)])
    sig("eshkol_b200_prepared_b_token", u64, [])
    sig("eshkol_b200_transfer_bytes", None, [ctypes.POINTER(u64), ctypes.POINTER(u64)])
    sig("eshkol_b200_last_gemm_ms", ctypes.c_double, [])
    sig("eshkol_gpu_set_residency", None, [ctypes.c_int, ctypes.c_size_t])
    sig("eshkol_gpu_invalidate", None, [vp, ctypes.c_size_t])
    sig("eshkol_gpu_residency_clear", None, [])
    sig("eshkol_rt_conv2d", vp, [vp, vp, vp, i64, i64])
    sig("eshkol_b200_set_tensor_allocator", None, [vp])
    sig("eshkol_b200_debug_gemm_model", None, [ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)])
    sig("eshkol_b200_debug_gemm_calibrate", None, [ctypes.c_int, ctypes.c_double, ctypes.c_double])
    sig("eshkol_b200_debug_set_wait_limit_ns", None, [ctypes.c_ulonglong])
    sig("eshkol_b200_debug_withhold_arrival", None, [ctypes.c_int])
    sig("eshkol_b200_sharded_open", ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, u64, u64, u64, ctypes.c_int,
                                                   ctypes.POINTER(vp)])
    sig("eshkol_b200_sharded_rows", ctypes.c_int, [vp, ctypes.POINTER(u64), ctypes.POINTER(u64)])
    sig("eshkol_b200_sharded_b_buffer", vp, [vp])
    sig("eshkol_b200_sharded_c_buffer", vp, [vp])
    sig("eshkol_b200_sharded_step", ctypes.c_int, [vp, vp])
    sig("eshkol_b200_sharded_close", ctypes.c_int, [vp])
    sig("eshkol_b200_debug_rendezvous", ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                       ctypes.c_int, ctypes.c_double])
    sig("eshkol_b200_debug_fail_allocation", None, [ctypes.c_int])
    sig("eshkol_b200_debug_sharded_plan", ctypes.c_int, [u64, ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_int]
        + [ctypes.POINTER(u64)] * 4)
    sig("eshkol_b200_debug_fetch", ctypes.c_int, [ctypes.c_int, ctypes.c_int, vp, u64, ctypes.POINTER(u64)])
    sig("eshkol_b200_debug_choose_tier", None, [u64, u64, u64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)])
    _lib = lib
    return lib
