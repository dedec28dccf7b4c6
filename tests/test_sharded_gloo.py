"""Row-sharded GEMM driver on CPU: world_size 2 and 3 over gloo, shard compute by the oracle.

Checks the host logic of the multi-GPU path (partition, broadcast of B, gather of C,
uneven row counts) and the property the design rests on: a row shard computed alone
has the bits of the same rows of the full product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eshkol_b200 import inputs
from eshkol_b200.sharded import ShardedGemm, row_partition
import oracle_lib as ol


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, K, N, out_path, panels):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A = inputs.full53(1, (M, K))
        B = inputs.full53(2, (K, N))

        def oracle_gemm(a, b, c):
            c.copy_(torch.from_numpy(ol.oz2_exact(a.numpy(), b.numpy(), 52)))

        sg = ShardedGemm(M, K, N, "cpu", gemm=oracle_gemm, panels=panels)
        r0, rows = sg.parts[rank]
        a_rows = torch.from_numpy(np.ascontiguousarray(A[r0:r0 + rows]))
        for _ in range(2):  # twice: the buffers are reused
            sg.step(a_rows, torch.from_numpy(B) if rank == 0 else None)
        C = sg.result().numpy()
        if rank == 0:
            np.save(out_path, C)
        # every rank holds the same gathered result
        t = torch.from_numpy(C.copy())
        dist.broadcast(t, src=0)
        assert np.array_equal(t.numpy().view(np.uint64), C.view(np.uint64))
    finally:
        dist.destroy_process_group()


def test_row_partition():
    assert row_partition(8, 2) == [(0, 4), (4, 4)]
    assert row_partition(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert row_partition(2, 3) == [(0, 1), (1, 1), (2, 0)]
    assert sum(r for _, r in row_partition(32768, 8)) == 32768


@pytest.mark.parametrize("world,M,panels", [(2, 64, 1), (3, 50, 4)])
def test_sharded_product_equals_unsharded_bits(tmp_path, world, M, panels):
    K, N = 300, 40
    out = str(tmp_path / "c.npy")
    mp.spawn(_worker, args=(world, _free_port(), M, K, N, out, panels), nprocs=world, join=True)
    C = np.load(out)
    full = ol.oz2_exact(inputs.full53(1, (M, K)), inputs.full53(2, (K, N)), 52)
    assert np.array_equal(C.view(np.uint64), full.view(np.uint64))


def test_transport_argument():
    """Off a GPU the copy-engine transport is not available: the driver keeps the collectives;
    a name it does not know is refused."""
    def gemm(a, b, c):
        c.copy_(a @ b)

    sg = ShardedGemm(8, 4, 6, "cpu", gemm=gemm, panels=2, transport="copy_engine")
    assert sg.transport == "collectives"
    A = torch.arange(32, dtype=torch.float64).reshape(8, 4)
    B = torch.arange(24, dtype=torch.float64).reshape(4, 6)
    assert torch.equal(sg.step(A, B), A @ B)
    with pytest.raises(ValueError):
        ShardedGemm(8, 4, 6, "cpu", gemm=gemm, transport="carrier-pigeon")


def _rendezvous_worker(name, rank, world, barriers, fail_at, leave_at, timeout_s, q):
    import ctypes
    import eshkol_b200 as eb
    lib = ctypes.CDLL(eb.library_path())
    lib.eshkol_b200_debug_rendezvous.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_double]
    import time
    t0 = time.perf_counter()
    rc = lib.eshkol_b200_debug_rendezvous(name.encode(), rank, world, barriers, fail_at, leave_at, timeout_s)
    q.put((rank, rc, time.perf_counter() - t0))


def _run_rendezvous(world, barriers, fail_rank=-1, fail_at=-1, leave_rank=-1, leave_at=-1, timeout_s=2.0):
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    name = f"/eshkol-b200-cputest-{os.getpid()}-{_free_port()}"
    procs = [ctx.Process(target=_rendezvous_worker,
                         args=(name, r, world, barriers, fail_at if r == fail_rank else -1,
                               leave_at if r == leave_rank else -1, timeout_s, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = dict()
    for _ in procs:
        r, rc, dt = q.get(timeout=60)
        out[r] = (rc, dt)
    for p in procs:
        p.join(timeout=30)
    try:
        os.unlink("/dev/shm" + name)
    except OSError:
        pass
    return out


def test_c_session_barriers_all_ranks_arrive():
    """The shared-memory rendezvous of the C multi-GPU driver (include/eshkol_b200_multi.h), without
    any GPU: four processes meet in the segment and pass 200 barriers."""
    out = _run_rendezvous(4, 200)
    assert all(rc == 0 for rc, _ in out.values()), out


def test_c_session_a_failed_rank_releases_the_others_at_once():
    """A rank whose step hit an error marks the session failed and leaves; the others' next
    barrier returns -1 instead of waiting for it (host-side failure detection: nothing on a GPU
    is made to fail)."""
    out = _run_rendezvous(3, 50, fail_rank=1, fail_at=20, timeout_s=20.0)
    assert all(rc == -1 for rc, _ in out.values()), out
    assert all(dt < 10.0 for _, dt in out.values()), out  # well before the 20 s timeout


def test_c_session_a_rank_that_leaves_is_noticed_by_timeout():
    """A rank that leaves between steps without a word: the others' barrier gives up after its
    timeout and returns -1; the rank that left saw no error."""
    out = _run_rendezvous(3, 50, leave_rank=2, leave_at=10, timeout_s=1.5)
    assert out[2][0] == 0
    assert out[0][0] == -1 and out[1][0] == -1
    assert all(1.0 < out[r][1] < 20.0 for r in (0, 1)), out


def test_column_shares_cover_the_panel_and_lighten_the_source():
    """The shares of a panel's columns are contiguous, in rank order and complete; the source
    rank's share is the stated fraction of the others' (none at weight 0, equal at weight 1)."""
    from eshkol_b200.sharded import column_shares
    for width, world, src, w in [(5120, 8, 0, 0.5), (1024, 8, 3, 0.5), (4096, 4, 0, 0.0), (4096, 4, 1, 1.0),
                                 (1000, 3, 2, 0.25), (7, 8, 0, 0.5), (256, 1, 0, 0.5)]:
        parts = column_shares(width, world, src, w)
        assert len(parts) == world
        assert parts[0][0] == 0 and sum(n for _, n in parts) == width
        for (a, n), (b, _) in zip(parts, parts[1:]):
            assert a + n == b
        if world > 1:
            others = [n for r, (_, n) in enumerate(parts) if r != src]
            assert max(others) - min(others) <= 1
            if w == 0.0:
                assert parts[src][1] == 0
            if w == 1.0:
                assert abs(parts[src][1] - others[0]) <= 1
            if 0.0 < w < 1.0 and width >= 64 * world:
                assert abs(parts[src][1] - w * others[0]) <= 1 + w


def test_the_c_driver_and_the_python_driver_follow_the_same_plan():
    """The schedule exists twice, in C (b200_sharded.cu) and over torch.distributed (sharded.py):
    both cut B into the same column panels and give every rank the same share of each."""
    import ctypes
    import eshkol_b200 as eb
    from eshkol_b200.sharded import column_shares, panel_columns
    lib = eb.load_library()
    u64 = ctypes.c_uint64
    for N, world, src, w in [(32768, 8, 0, 0.5), (32768, 4, 0, 0.5), (32768, 2, 1, 1.0), (8192, 8, 3, 0.0),
                             (16384, 4, 0, 0.25), (1000, 4, 0, 0.5), (4096, 1, 0, 0.5)]:
        col0, width = (u64 * 24)(), (u64 * 24)()
        first, count = (u64 * (24 * world))(), (u64 * (24 * world))()
        P = lib.eshkol_b200_debug_sharded_plan(N, world, src, w, 24, col0, width, first, count)
        want = panel_columns(N, 4, "gentle")
        assert P == len(want), (N, world)
        assert [(int(col0[p]), int(width[p])) for p in range(P)] == want
        for p, (_, wd) in enumerate(want):
            shares = column_shares(wd, world, src, w)
            assert [(int(first[p * world + r]), int(count[p * world + r])) for r in range(world)] == shares
