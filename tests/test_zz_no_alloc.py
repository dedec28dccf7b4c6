"""The allocation-free GEMM entry point against the ordinary one.

Some hosts cannot let a matmul allocate device memory: their own arena already
holds all of it, or they run other streams that a cudaMalloc would stall.  For
them the library keeps a fixed scratch array and offers
eshkol_b200_gemm_f64_static_scratch.  This file checks, through the C ABI, that
it returns the same bits as eshkol_b200_gemm_f64_device on two calls in a row
(the second smaller, so stale contents of the shared array would show), and that
it refuses a shape the array cannot serve.  It is collected last on purpose.
"""
import numpy as np
import pytest

import eshkol_b200 as eb
from eshkol_b200 import api, inputs
import gpu_util as gu

pytestmark = pytest.mark.gpu


def _static_gemm(lib, A, B):
    import torch
    dA = torch.from_numpy(np.ascontiguousarray(A)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B)).cuda()
    dC = torch.full((A.shape[0], B.shape[1]), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    rc = lib.eshkol_b200_gemm_f64_static_scratch(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                                                 A.shape[0], A.shape[1], B.shape[1])
    assert rc == 0
    assert api.sync_status() == 0
    return dC.cpu().numpy()


def test_static_scratch_gemm_matches_the_allocating_entry_point_twice(gpu_lib):
    first = (inputs.full53(21, (384, 1500)), inputs.full53(22, (1500, 300)))
    second = (inputs.wide(23, (130, 700), span=9, lo=-4), inputs.uniform(24, (700, 257)))
    for A, B in (first, second):
        got = _static_gemm(gpu_lib, A, B)
        want = gu.gemm(A, B)  # eshkol_b200_gemm_f64_device, exact tier
        assert gu.same_bits(got, want)  # tolerance of the exact-tier tests: none


def test_static_scratch_gemm_takes_no_device_memory(gpu_lib):
    """What the entry point is for: between the moment the caller's buffers exist and the
    moment the result is there, neither the driver's free-memory figure nor the library's own
    workspace may move -- the scratch array was taken when eshkol_b200_init loaded it."""
    import torch
    A = torch.from_numpy(inputs.uniform(31, (256, 900))).cuda()
    B = torch.from_numpy(inputs.uniform(32, (900, 256))).cuda()
    C = torch.empty((256, 256), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    ws0 = api.load_library().eshkol_b200_workspace_bytes()
    for _ in range(2):
        assert gpu_lib.eshkol_b200_gemm_f64_static_scratch(A.data_ptr(), B.data_ptr(), C.data_ptr(), 256, 900, 256) == 0
        assert api.sync_status() == 0
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0
        assert api.load_library().eshkol_b200_workspace_bytes() == ws0
    assert gu.same_bits(C.cpu().numpy(), gu.gemm(A.cpu().numpy(), B.cpu().numpy()))


def test_static_scratch_gemm_refuses_what_the_array_cannot_hold(gpu_lib):
    import torch
    n = 2048  # needs far more than the 24 MiB array
    a = torch.zeros((n, n), dtype=torch.float64, device="cuda")
    c = torch.zeros((n, n), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    assert gpu_lib.eshkol_b200_gemm_f64_static_scratch(a.data_ptr(), a.data_ptr(), c.data_ptr(), n, n, n) == -1
    assert api.sync_status() == 0
