"""Row-sharded f64 GEMM across the GPUs of one box (one process per GPU).

Rows of A are independent in every tier: the scale of row i, its residues and
C[i, :] depend on row i, on B and on the global exponent E only (E = 52 whenever
K <= 131071), so a row shard computed alone carries the same bits as the same rows
of the full product.  Rank r owns a contiguous block of rows of A and of C; B is
broadcast from one rank and the blocks of C are all-gathered, both with
torch.distributed (NCCL over NVLink on GPUs, gloo in the CPU tests).  The reference
has no multi-device code; this is the sharding the 32768^3 row-sharded configuration asks for.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Optional

import torch
import torch.distributed as dist


def panel_columns(N: int, panels: int, taper) -> list[tuple[int, int]]:
    """(first column, width) of every column panel of B.

    taper False / None: `panels` equal panels.  "half": a first and a last panel of half the
    width.  "geometric": widths w/8, w/4, w/2 at either end (w = N / panels) and the rest in
    panels - 2 (at least one) equal middle panels -- the first panel's way to the ranks and the
    last panel's way back are the two transfers no products hide, and a panel only has to arrive
    before the products of the one before it end, which a doubling of the width still allows
    (moving a column costs about a third of multiplying by it).  Widths stay multiples of 256
    (the products kernel's tile); a shape that does not allow that gets equal panels."""
    if panels <= 0 or N % panels != 0:
        panels = 1
    w = N // panels
    equal = [(p * w, w) for p in range(panels)]
    if taper in (True, "half") and panels >= 2 and w % 512 == 0:
        h = w // 2
        return [(0, h)] + [(h + i * w, w) for i in range(panels - 1)] + [(N - h, h)]
    if taper == "gentle" and panels >= 2 and w % 2048 == 0:
        # widths grow by half from w/8 (a panel of residue planes is twice the bytes of its f64
        # columns, so its exchange hides behind the products of the panel before it only up to a
        # ratio of about 1.5), stay at about w, and halve down to w/8 at the end
        up, x = [], w // 8
        while x < w * 3 // 4:
            up.append(x)
            x = (x * 3 // 2 + 255) // 256 * 256
        down = [w // 2, w // 4, w // 8]
        mid_total = N - sum(up) - sum(down)
        n_mid = max(1, -(-mid_total // w))
        mid = (mid_total // n_mid) // 256 * 256
        if mid <= 0:
            return equal
        widths = up + [mid] * (n_mid - 1) + [mid_total - mid * (n_mid - 1)] + down
        out, c0 = [], 0
        for wd in widths:
            out.append((c0, wd))
            c0 += wd
        return out
    if taper == "geometric" and panels >= 2 and w % 2048 == 0:
        ramp = [w // 8, w // 4, w // 2]
        mid_total = N - 2 * sum(ramp)
        n_mid = max(1, panels - 2)
        mid = (mid_total // n_mid) // 256 * 256
        if mid <= 0:
            return equal
        widths = ramp + [mid] * (n_mid - 1) + [mid_total - mid * (n_mid - 1)] + ramp[::-1]
        out, c0 = [], 0
        for wd in widths:
            out.append((c0, wd))
            c0 += wd
        return out
    return equal


def row_partition(M: int, world: int) -> list[tuple[int, int]]:
    """(first row, row count) per rank: contiguous blocks, sizes differing by at most one."""
    base, extra = divmod(M, world)
    out, start = [], 0
    for r in range(world):
        rows = base + (1 if r < extra else 0)
        out.append((start, rows))
        start += rows
    return out


def column_shares(width: int, world: int, src: int, src_weight: float) -> list[tuple[int, int]]:
    """(first column, column count) per rank of one panel, contiguous, in rank order.  The source
    rank also sends every other rank its f64 columns, so its link carries more than the others';
    its share (and with it the planes it serves to every peer) is src_weight of theirs."""
    if world == 1:
        return [(0, width)]
    n0 = min(width, max(0, int(width * src_weight / (world - 1 + src_weight))))
    base, extra = divmod(width - n0, world - 1)
    out, start, k = [], 0, 0
    for r in range(world):
        if r == src:
            n = n0
        else:
            n = base + (1 if k < extra else 0)
            k += 1
        out.append((start, n))
        start += n
    return out


class CShardedGemm:
    """The same sharded product driven entirely from C (include/eshkol_b200_multi.h): the ranks
    meet in a POSIX shared-memory segment, which carries the CUDA IPC handles and the host
    barriers, so a host that is not Python can do exactly this.  This class only adapts the C
    handle to the surface of ShardedGemm that the benchmark and the tests use; `name` must be the
    same fresh string on every rank (torch.distributed, when initialised, is used for nothing but
    agreeing on it)."""

    transport = "copy_engine (C driver, shared-memory rendezvous)"
    split_shared = True
    b_in_place = True

    def __init__(self, M: int, K: int, N: int, device, *, rank: int = 0, world: int = 1, src: int = 0,
                 name: Optional[str] = None):
        from . import api
        self.api = api
        self.lib = api.load_library()
        self.M, self.K, self.N = M, K, N
        self.rank, self.world, self.src = rank, world, src
        self.device = torch.device(device)
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        if self.lib.eshkol_b200_init(index) != 0:
            raise RuntimeError("eshkol_b200_init failed: no usable sm_100 device")
        if name is None:
            import os
            token = [os.getpid() if rank == 0 else 0]
            if world > 1:
                dist.broadcast_object_list(token, src=0)
            name = f"/eshkol-b200-{token[0]}"
        self.name = name
        handle = ctypes.c_void_p()
        if self.lib.eshkol_b200_sharded_open(name.encode(), rank, world, M, K, N, src, ctypes.byref(handle)) != 0:
            raise RuntimeError("eshkol_b200_sharded_open failed")
        self._h = handle
        r0, rr = ctypes.c_uint64(), ctypes.c_uint64()
        self.lib.eshkol_b200_sharded_rows(self._h, ctypes.byref(r0), ctypes.byref(rr))
        self.row0, self.rows = int(r0.value), int(rr.value)
        self.parts = row_partition(M, world)
        self.cols = panel_columns(N, 4, "gentle")
        self.panels = len(self.cols)
        self.C = self._view(self.lib.eshkol_b200_sharded_c_buffer(self._h), (M, N))
        b = self.lib.eshkol_b200_sharded_b_buffer(self._h)
        self._B = self._view(b, (K, N)) if b else None

    def _view(self, ptr: int, shape) -> torch.Tensor:
        class _Block:
            pass
        blk = _Block()
        blk.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f8", "data": (int(ptr), False),
                                        "version": 2, "strides": None}
        return torch.as_tensor(blk, device=self.device)

    def source_buffer(self) -> Optional[torch.Tensor]:
        return self._B

    def step(self, A_rows: torch.Tensor, B_src: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.rank == self.src and (B_src is None or B_src.data_ptr() != self._B.data_ptr()):
            raise ValueError("the source rank must pass the tensor source_buffer() returned")
        if A_rows.shape != (self.rows, self.K) or not A_rows.is_contiguous():
            raise ValueError(f"rank {self.rank} expects {self.rows} x {self.K} contiguous rows of A")
        torch.cuda.current_stream(self.device).synchronize()  # A (and B) are complete before the call
        if self.lib.eshkol_b200_sharded_step(self._h, A_rows.data_ptr()) != 0:
            raise RuntimeError("eshkol_b200_sharded_step failed")
        return self.C

    def close(self) -> None:
        if self._h is not None:
            self.C = self._B = None
            self.lib.eshkol_b200_sharded_close(self._h)
            self._h = None


class _DeviceBackend:
    """The library's device GEMM, with both operands prepared separately when the exact
    tier allows it: A once per step, each column panel of B as it arrives.  The library
    launches on its own stream; `stream` wraps it for torch so that the two sides are ordered
    by events on the device and the host never waits inside a step."""

    on_device = True

    def __init__(self, tier: int, param: int, device, comm_sms: int = 0):
        from . import api
        self.api = api
        self.lib = api.load_library()
        self.tier, self.param = tier, param
        self.prepared = tier == 0 and param in (0, 16)
        # the stream handle is null until the library is initialised, and a null handle would
        # wrap the legacy default stream: every ordering below would then order the wrong stream
        index = torch.device(device).index
        if index is None:
            index = torch.cuda.current_device()
        if self.lib.eshkol_b200_init(index) != 0:
            raise RuntimeError("eshkol_b200_init failed: no usable sm_100 device")
        if not api.stream_handle():
            raise RuntimeError("the library reports no stream after eshkol_b200_init")
        self.stream = torch.cuda.ExternalStream(api.stream_handle(), device=device)
        if comm_sms > 0:
            # the persistent products kernels leave these SMs to the collectives' kernels
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            self.lib.eshkol_b200_set_sm_limit(max(2, sms - comm_sms))

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc})")

    def begin(self, a: torch.Tensor, panel_cols: int) -> None:
        if self.prepared:
            self._check(self.lib.eshkol_b200_prepare_a_f64_device(a.data_ptr(), a.shape[0], a.shape[1], panel_cols),
                        "prepare_a")

    def panel(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> None:
        """c: rows x panel-width view, contiguous or a column panel of a wider row-major matrix"""
        ldc = 0 if c.is_contiguous() else c.stride(0)
        opts = self.api.make_opts(self.tier, self.param, ldc=ldc)
        if self.prepared:
            self._check(self.lib.eshkol_b200_prepare_b_f64_device(b.data_ptr(), b.shape[0], b.shape[1]), "prepare_b")
            self._check(self.lib.eshkol_b200_multiply_prepared_f64_device(c.data_ptr(), ctypes.byref(opts)), "multiply")
        else:
            self.api.gemm_device(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape[0], a.shape[1], b.shape[1], opts)

    def finish(self) -> None:
        st = self.api.sync_status()
        if st != 0:
            raise RuntimeError(f"GEMM kernel status {st}")


class _CallableBackend:
    """gemm(a_rows, b_panel, c_panel) supplied by the caller (CPU tests)."""

    on_device = False

    def __init__(self, fn: Callable):
        self.fn = fn

    def begin(self, a, panel_cols) -> None:
        pass

    def panel(self, a, b, c) -> None:
        self.fn(a, b, c)

    def finish(self) -> None:
        pass


class ShardedGemm:
    """Buffers and schedule of one sharded product C = A @ B with A row-sharded.

    B travels in `panels` column panels (contiguous K x N/panels blocks packed on the
    source rank): every panel's transfer is enqueued at once, each panel is multiplied as soon
    as it has arrived, and its block of C travels to the other ranks while the next panel is
    being multiplied, so only the first panel's way out and the last one's way back are
    exposed.  All buffers are allocated once; step() allocates nothing.

    transport: "collectives" moves the panels with torch.distributed (broadcast, all-gather:
    NCCL on GPUs, gloo in the CPU tests); "copy_engine" (GPUs only) with the library's copy
    engine entry points over CUDA IPC, which run beside the products kernels where a
    collective's kernel has to wait for the gaps between them.  If the peers' memory cannot
    be opened the constructor says so and falls back to the collectives on every rank.

    comm_sms: SMs the products kernels leave free for the collectives.  A products CTA fills
    its SM's shared memory, so a collective's kernel launched beside them would otherwise
    wait for the gap between two products kernels on every rank; the process group should be
    created with as many CTAs at most (NCCL_MAX_CTAS).
    """

    def __init__(self, M: int, K: int, N: int, device, *, tier: int = 0, param: int = 0, src: int = 0,
                 group=None, gemm: Optional[Callable] = None, panels: int = 1, comm_sms: int = 0,
                 transport: str = "collectives", taper=False, share_split: bool = False, b_in_place: bool = False):
        self.M, self.K, self.N = M, K, N
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.src = src
        self.parts = row_partition(M, self.world)
        self.row0, self.rows = self.parts[self.rank]
        self.max_rows = max(r for _, r in self.parts)
        self.device = torch.device(device)
        self.backend = _CallableBackend(gemm) if gemm is not None else _DeviceBackend(tier, param, self.device, comm_sms if self.world > 1 else 0)
        self._side = None
        self.trace = None  # set to [] to collect (label, CUDA event) marks of the next step
        self.host_trace = []  # (label, host seconds) of the traced step
        self.panels = panels if (panels > 0 and N % panels == 0) else 1
        self.width = N // self.panels
        # column range of every panel: equal widths, or (copy-engine transport only) narrower
        # panels at either end (panel_columns)
        self.cols = [(p * self.width, self.width) for p in range(self.panels)]
        self._taper_wanted = taper if self.panels >= 2 else False
        if transport not in ("collectives", "copy_engine"):
            raise ValueError(f"unknown transport {transport!r}")
        self.transport = "collectives"
        self.Cp = None
        # share_split (copy-engine transport): every rank scans and splits 1/world of a panel's
        # columns and the ranks exchange the residue planes, instead of every rank splitting all of B
        self.split_shared = False
        self._share_wanted = bool(share_split)
        # b_in_place (with share_split): the source keeps B in source_buffer() and nothing is packed
        self.b_in_place = bool(b_in_place) and bool(share_split)
        # share_split: how many panels beyond the one being multiplied have their shares split
        # (and, a host barrier later, their planes on the way)
        self.ahead = max(2, int(os.environ.get("ESHKOL_B200_AHEAD", "2") or 2))
        if transport == "copy_engine" and self.world > 1 and self.backend.on_device:
            # the panel buffer of B and C itself are library allocations the peers open; products
            # write their block of C in place and the peers pull it from there
            import datetime
            import sys
            self.ctl = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=180))
            uniform = (self.panels, self.width, self.cols)
            if self._taper_wanted:
                self.cols = panel_columns(N, self.panels, self._taper_wanted)
                self.panels = len(self.cols)
            try:
                self._open_peers()
                opened = 1
            except RuntimeError as exc:
                sys.stderr.write(f"[eshkol-b200] rank {self.rank}: copy-engine transport unavailable ({exc})\n")
                opened = 0
            agreed = torch.tensor([opened], dtype=torch.int32)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.ctl)
            if int(agreed.item()) == 1:
                self.transport = "copy_engine"
            else:
                # falling back together: give back whatever was opened or made on the way
                self._closed = False
                self.close()
                self._closed = False
                self.panels, self.width, self.cols = uniform
        if self.transport != "copy_engine":
            # panel-major copy of B: panel p is the contiguous K x width block of columns p*width ...
            self.Bp = torch.empty((self.panels, K, self.width), dtype=torch.float64, device=self.device)
            self.C = torch.empty((M, N), dtype=torch.float64, device=self.device)
            # gathered blocks: [panel][rank][row][column in panel]; padding rows are never read back
            self.Cp = torch.empty((self.panels, self.world, self.max_rows, self.width), dtype=torch.float64,
                                  device=self.device)

    # ------------------------------------------------------------ copy-engine transport
    class _DeviceBlock:
        """A cudaMalloc block owned by the library, visible to torch as a tensor."""

        def __init__(self, lib, shape, device):
            self.lib = lib
            n = 1
            for d in shape:
                n *= d
            ptr = ctypes.c_void_p()
            if lib.eshkol_b200_mem_alloc(0, n * 8, ctypes.byref(ptr)) != 0:
                raise RuntimeError(f"allocation of {n * 8} bytes failed")
            self.ptr = ptr.value
            self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f8", "data": (self.ptr, False),
                                             "version": 2, "strides": None}
            self.tensor = torch.as_tensor(self, device=device)

        def free(self) -> None:
            if self.ptr:
                self.tensor = None
                self.lib.eshkol_b200_mem_free(0, self.ptr)
                self.ptr = 0

        def handle(self) -> bytes:
            buf = ctypes.create_string_buffer(64)
            if self.lib.eshkol_b200_ipc_export_mem(self.ptr, buf) != 0:
                raise RuntimeError("ipc_export_mem failed")
            return buf.raw

    def _open_peers(self) -> None:
        """Every rank opens every other rank's B-panel buffer and C (CUDA IPC memory handles,
        opened in the rank's own context) and its hand-off events (interprocess events).  Data
        then moves by copy-engine pulls over NVLink, ordered on the device by those events; a
        gloo barrier only makes sure an event's record has been *called* before a peer calls
        wait on it (the host runs far ahead of the device).

        Every rank takes part in every exchange whatever failed locally (a rank that stopped
        half-way would leave the others waiting); the first failure is raised at the end."""
        lib = self.backend.lib
        W, R, P = self.world, self.rank, self.panels
        failure = []

        def attempt(fn, *args):
            if failure:
                return None
            try:
                return fn(*args)
            except RuntimeError as exc:
                failure.append(str(exc))
                return None

        def exchange(obj):
            objs = [None] * W
            dist.all_gather_object(objs, obj, group=self.ctl)
            return objs

        def import_mem(handle: bytes) -> int:
            out = ctypes.c_void_p()
            if handle is None or lib.eshkol_b200_ipc_import_mem(handle, ctypes.byref(out)) != 0:
                raise RuntimeError("a peer's memory could not be opened (no peer access between the GPUs?)")
            return out.value

        def make_blocks():
            self._blk_B = self._DeviceBlock(lib, (self.K * self.N,), self.device)
            self._blk_C = self._DeviceBlock(lib, (self.M, self.N), self.device)
            return (self._blk_B.handle(), self._blk_C.handle())

        mine = attempt(make_blocks)
        hs = exchange(mine)
        # base addresses of every rank's Bp and C in this process (own rank: the local pointer)
        self._addr_B = [None] * W
        self._addr_C = [None] * W
        for q in range(W):
            if q == R:
                if mine is not None:
                    self._addr_B[q], self._addr_C[q] = self._blk_B.ptr, self._blk_C.ptr
            elif hs[q] is None:
                failure.append(f"rank {q} exported nothing")
            else:
                self._addr_B[q] = attempt(import_mem, hs[q][0])
                self._addr_C[q] = attempt(import_mem, hs[q][1])

        def create_events(n: int):
            evs, handles = [], []
            for _ in range(n):
                ev, buf = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                if lib.eshkol_b200_ipc_event_create(ctypes.byref(ev), buf) != 0:
                    raise RuntimeError("an interprocess event could not be created")
                evs.append(ev.value)
                handles.append(buf.raw)
            return evs, handles

        def import_event(h: bytes) -> int:
            ev = ctypes.c_void_p()
            if lib.eshkol_b200_ipc_event_import(h, ctypes.byref(ev)) != 0:
                raise RuntimeError("a peer's event could not be opened")
            return ev.value

        def make_events(n: int):
            made = attempt(create_events, n)
            theirs = exchange(None if made is None else made[1])
            table = []
            for q in range(W):
                if q == R:
                    table.append(None if made is None else made[0])
                elif theirs[q] is None:
                    failure.append(f"rank {q} exported no events")
                    table.append(None)
                else:
                    table.append([attempt(import_event, h) for h in theirs[q]])
            return table

        self._ev_packed = make_events(P)   # on the source rank: panel p packed
        self._ev_slice = make_events(P)    # this rank's K-slice of panel p is in its Bp
        self._ev_block = make_events(P)    # this rank's block of C, panel p, is computed
        if self._share_wanted and self.backend.prepared:
            # one buffer of residue planes per panel (the whole prepared B stays resident: 16.3
            # bytes per element), opened by every peer; this rank writes its share of the columns
            def make_planes():
                self._blk_P = [self._DeviceBlock(lib, (int(lib.eshkol_b200_prepared_b_bytes(self.K, wd) + 7) // 8,),
                                                 self.device) for _, wd in self.cols]
                return [b.handle() for b in self._blk_P]
            mine_p = attempt(make_planes)
            hp = exchange(mine_p)
            self._addr_P = [None] * W
            for q in range(W):
                if q == R:
                    if mine_p is not None:
                        self._addr_P[q] = [b.ptr for b in self._blk_P]
                elif hp[q] is None:
                    failure.append(f"rank {q} exported no plane buffers")
                else:
                    self._addr_P[q] = [attempt(import_mem, h) for h in hp[q]]
            self._ev_planes = make_events(P)   # this rank's columns of panel p are split
            w_src = min(1.0, max(0.0, float(os.environ.get("ESHKOL_B200_SRC_SHARE", "0.5") or 0.5)))
            self._cparts = [column_shares(wd, W, self.src, w_src) for _, wd in self.cols]
            self._regions = []
            for p, (_, wd) in enumerate(self.cols):
                per_rank = []
                for q in range(W):
                    c0, n = self._cparts[p][q]
                    out = (ctypes.c_uint64 * 28)()
                    if n and lib.eshkol_b200_prepared_b_regions(self.K, wd, c0, n, out) != 7:
                        failure.append("prepared_b_regions failed")
                    per_rank.append([tuple(int(out[4 * i + j]) for j in range(4)) for i in range(7)] if n else [])
                self._regions.append(per_rank)
            if not failure:
                ncmax = max(n for parts in self._cparts for _, n in parts)
                # this rank's f64 columns of the panels in flight (the source reads its own B in place)
                self._bcol = [torch.empty((self.K, ncmax), dtype=torch.float64, device=self.device) for _ in range(3)]
                self.split_shared = True
        if failure:
            raise RuntimeError(failure[0])
        flat = self._blk_B.tensor
        # panel p: the contiguous K x width block of its columns, packed one panel after the other
        self.Bp = [flat[self.K * c0:self.K * (c0 + wd)].view(self.K, wd) for c0, wd in self.cols]
        self.C = self._blk_C.tensor
        self._x1 = torch.cuda.Stream(self.device)
        self._x2 = torch.cuda.Stream(self.device)
        n_pool = min(8, max(1, int(os.environ.get("ESHKOL_B200_POOL", "4") or 4)))
        self._pull_streams = [torch.cuda.Stream(self.device) for _ in range(min(n_pool, max(1, W - 1)))]
        # The blocks of C move on streams of their own.  With the planes of several panels on
        # their way ahead of the products (self.ahead) the block copies no longer take the copy
        # engines from planes the products are about to need.
        self._gather_streams = [torch.cuda.Stream(self.device) for _ in self._pull_streams]
        self._k_parts = row_partition(self.K, W)
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        """Give back what the constructor took: imported peer memory is closed, the hand-off
        events destroyed and the two library blocks freed, after every rank has finished with
        them.  The object must not be used afterwards.  Every rank has to call it."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        if self.backend.on_device:
            torch.cuda.synchronize(self.device)
        ctl = getattr(self, "ctl", None)
        if ctl is not None:
            dist.barrier(group=ctl)  # no peer still reads this rank's blocks
        lib = getattr(self.backend, "lib", None)
        if lib is not None:
            for table in (getattr(self, "_addr_B", None), getattr(self, "_addr_C", None)):
                for q, addr in enumerate(table or []):
                    if addr and q != self.rank:
                        lib.eshkol_b200_ipc_close_mem(addr)
            for q, addrs in enumerate(getattr(self, "_addr_P", None) or []):
                if q != self.rank:
                    for addr in addrs or []:
                        if addr:
                            lib.eshkol_b200_ipc_close_mem(addr)
            for table in (getattr(self, "_ev_packed", None), getattr(self, "_ev_slice", None),
                          getattr(self, "_ev_block", None), getattr(self, "_ev_planes", None)):
                for evs in table or []:
                    for ev in evs or []:
                        if ev:
                            lib.eshkol_b200_event_destroy(ev)
            if ctl is not None:
                dist.barrier(group=ctl)  # every import is closed before its owner frees the memory
            self.Bp = self.C = None
            for name in ("_blk_B", "_blk_C"):
                blk = getattr(self, name, None)
                if blk is not None:
                    blk.free()
                    setattr(self, name, None)
            for blk in getattr(self, "_blk_P", None) or []:
                blk.free()
            self._blk_P = None
            self._bcol = None
        self._addr_B = self._addr_C = self._ev_packed = self._ev_slice = self._ev_block = None
        self._addr_P = self._ev_planes = None
        self.Bp = self.C = self.Cp = None

    def _record(self, ev: int, stream) -> None:
        if self.backend.lib.eshkol_b200_event_record(ev, stream.cuda_stream) != 0:
            raise RuntimeError("event_record failed")

    def _wait(self, ev: int, stream) -> None:
        if self.backend.lib.eshkol_b200_event_wait(ev, stream.cuda_stream) != 0:
            raise RuntimeError("event_wait failed")

    def _pull_b_slice(self, q_from: int, p: int, k0: int, kn: int, stream) -> None:
        """rows [k0, k0+kn) of panel p: rank q_from's Bp -> this rank's Bp (contiguous, one copy)"""
        c0, wd = self.cols[p]
        off = (self.K * c0 + k0 * wd) * 8
        rc = self.backend.lib.eshkol_b200_copy_async(self._addr_B[self.rank] + off, self._addr_B[q_from] + off,
                                                     kn * wd * 8, stream.cuda_stream)
        if rc != 0:
            raise RuntimeError("copy_async failed")

    def _pull_c_block(self, q: int, p: int, stream) -> None:
        """rank q's rows of the panel-p columns of C: its C -> the same place in this rank's C"""
        q0, rows_q = self.parts[q]
        c0, wd = self.cols[p]
        off = (q0 * self.N + c0) * 8
        rc = self.backend.lib.eshkol_b200_copy2d_async(self._addr_C[self.rank] + off, self.N * 8,
                                                       self._addr_C[q] + off, self.N * 8, wd * 8, rows_q,
                                                       stream.cuda_stream)
        if rc != 0:
            raise RuntimeError("copy2d_async failed")

    def _step_copy_engine(self, A_rows: torch.Tensor, B_src: Optional[torch.Tensor]) -> torch.Tensor:
        P, R, W = self.panels, self.rank, self.world
        cur = torch.cuda.current_stream(self.device)
        lib = self.backend.stream
        if self._side is None:
            self._side = torch.cuda.Stream(self.device)
        x1, x2, xo = self._x1, self._x2, self._side
        self._mark("start", cur)
        for st in (x1, x2, xo, *self._pull_streams):
            st.wait_stream(cur)
        if self.rows:
            lib.wait_stream(cur)
            self.backend.begin(A_rows, max(wd for _, wd in self.cols))
            self._mark("A prepared", lib)
        # B: the source packs a panel; every rank pulls its own K-slice of it from the source
        # (phase 1, the source's egress carries the panel once), then the other slices from
        # the ranks that hold them (phase 2)
        if R == self.src:
            if not (B_src.is_contiguous() and B_src.shape == (self.K, self.N)):
                raise ValueError("B must be a contiguous K x N matrix")
            # packed by the copy engines (about 0.9 TB/s on an idle GPU): an elementwise kernel of
            # another stream would wait for the gaps between the products kernels
            st = x1
            for p, (c0, wd) in enumerate(self.cols):
                rc = self.backend.lib.eshkol_b200_copy2d_async(
                    self._addr_B[R] + self.K * c0 * 8, wd * 8, B_src.data_ptr() + c0 * 8, self.N * 8,
                    wd * 8, self.K, st.cuda_stream)
                if rc != 0:
                    raise RuntimeError("copy2d_async failed")
                self._mark(f"packed {p}", st)
                self._record(self._ev_packed[R][p], st)
                self._record(self._ev_slice[R][p], st)
        dist.barrier(group=self.ctl)
        k0, kn = self._k_parts[R]
        if R != self.src:
            for p in range(P):
                self._wait(self._ev_packed[self.src][p], x1)
                self._pull_b_slice(self.src, p, k0, kn, x1)
                self._mark(f"own slice {p}", x1)
                self._record(self._ev_slice[R][p], x1)
        dist.barrier(group=self.ctl)
        arrived = []
        for p in range(P):
            if R != self.src:
                for i in range(1, W):
                    q = (R + i) % W
                    q0, qn = self._k_parts[q]
                    self._wait(self._ev_slice[q][p], x2)
                    self._pull_b_slice(q, p, q0, qn, x2)
                self._wait(self._ev_slice[R][p], x2)
            else:
                self._wait(self._ev_packed[R][p], x2)
            ev = torch.cuda.Event()
            ev.record(x2)
            arrived.append(ev)
            self._mark(f"B panel {p} arrived", x2)
        for p in range(P):
            self._host_mark(f"pulls of {p} called")
            if self.rows:
                lib.wait_event(arrived[p])
                self._mark(f"panel {p} products start", lib)
                c0, wd = self.cols[p]
                self.backend.panel(A_rows, self.Bp[p], self.C[self.row0:self.row0 + self.rows, c0:c0 + wd])
                self._mark(f"panel {p} products done", lib)
            self._record(self._ev_block[R][p], lib)
        dist.barrier(group=self.ctl)
        # C: pull every other rank's block of a panel, straight into its place in C, once computed;
        # the pulls of a panel are spread over a few streams so that several copy engines work
        # at once (one 2-D pull alone runs far below the link rate)
        pool = self._pull_streams
        for p in range(P):
            for i in range(1, W):
                q = (R + i) % W
                if self.parts[q][1] == 0:
                    continue
                st = pool[i % len(pool)]
                self._wait(self._ev_block[q][p], st)
                self._pull_c_block(q, p, st)
            for st in pool:
                xo.wait_stream(st)
            self._mark(f"panel {p} gathered", xo)
        cur.wait_stream(lib)
        cur.wait_stream(xo)
        cur.wait_stream(x1)
        cur.wait_stream(x2)
        self.backend.finish()
        cur.synchronize()
        # nobody overwrites a buffer a peer may still be reading
        dist.barrier(group=self.ctl)
        return self.C

    def _copy2d(self, dst: int, dpitch: int, src: int, spitch: int, width: int, rows: int, stream) -> None:
        if self.backend.lib.eshkol_b200_copy2d_async(dst, dpitch, src, spitch, width, rows, stream.cuda_stream) != 0:
            raise RuntimeError("copy2d_async failed")

    def source_buffer(self) -> Optional[torch.Tensor]:
        """On the source rank: a K x N tensor inside the buffer the peers have opened.  A caller
        that keeps (or builds) B there and passes it to step() saves the source GPU the packing
        of every panel -- the peers then read their columns of B straight out of it."""
        if self.transport != "copy_engine" or self.rank != self.src or not self.split_shared:
            return None
        return self._blk_B.tensor[: self.K * self.N].view(self.K, self.N)

    def _step_shared_split(self, A_rows: torch.Tensor, B_src: Optional[torch.Tensor]) -> torch.Tensor:
        """The copy-engine step with the split of B shared: rank r scans and splits columns
        [c0_r, c0_r + n_r) of every panel (1/world of the work every rank did before) into its
        place of the panel's plane buffer and pulls the other ranks' pieces from their buffers.
        Host calls run two panels ahead of the products; one host barrier per panel orders the
        calls of an interprocess event's record before the peers' calls of its wait."""
        P, R, W = self.panels, self.rank, self.world
        lib_h = self.backend.lib
        cur = torch.cuda.current_stream(self.device)
        lib = self.backend.stream
        if self._side is None:
            self._side = torch.cuda.Stream(self.device)
        x1, x2, xo, pool, gpool = self._x1, self._x2, self._side, self._pull_streams, self._gather_streams
        self._mark("start", cur)
        for st in (x1, x2, xo, *pool, *gpool):
            st.wait_stream(cur)
        lib.wait_stream(cur)
        # B in place: the source's B already lies in the buffer the peers opened (row pitch N);
        # otherwise the source packs panel after panel into it (row pitch = the panel's width)
        direct = self.b_in_place
        if R == self.src:
            if not (B_src.is_contiguous() and B_src.shape == (self.K, self.N)):
                raise ValueError("B must be a contiguous K x N matrix")
            if direct and B_src.data_ptr() != self._blk_B.ptr:
                raise ValueError("b_in_place: the source rank must pass the tensor source_buffer() returned")
            for p, (c0, wd) in enumerate(self.cols):
                if not direct:
                    self._copy2d(self._addr_B[R] + self.K * c0 * 8, wd * 8, B_src.data_ptr() + c0 * 8, self.N * 8,
                                 wd * 8, self.K, x1)
                    self._mark(f"packed {p}", x1)
                self._record(self._ev_packed[R][p], x1)
        dist.barrier(group=self.ctl)
        bcol_free = [None] * len(self._bcol)

        def stage_prep(p: int) -> None:
            c0p, wd = self.cols[p]
            c0, n = self._cparts[p][R]
            if n:
                if R == self.src:
                    src_ptr, ldb = B_src.data_ptr() + (c0p + c0) * 8, self.N
                else:
                    slot = p % len(self._bcol)
                    if bcol_free[slot] is not None:
                        x1.wait_event(bcol_free[slot])  # the split that read this slot is through
                    self._wait(self._ev_packed[self.src][p], x1)
                    if direct:
                        self._copy2d(self._bcol[slot].data_ptr(), n * 8, self._addr_B[self.src] + (c0p + c0) * 8,
                                     self.N * 8, n * 8, self.K, x1)
                    else:
                        self._copy2d(self._bcol[slot].data_ptr(), n * 8,
                                     self._addr_B[self.src] + (self.K * c0p + c0) * 8, wd * 8, n * 8, self.K, x1)
                    got = torch.cuda.Event()
                    got.record(x1)
                    lib.wait_event(got)
                    src_ptr, ldb = self._bcol[slot].data_ptr(), n
                if lib_h.eshkol_b200_prepare_b_columns_f64_device(src_ptr, ldb, self.K, wd, c0, n, self._blk_P[p].ptr) != 0:
                    raise RuntimeError("prepare_b_columns failed")
                if R != self.src:
                    done = torch.cuda.Event()
                    done.record(lib)
                    bcol_free[p % len(self._bcol)] = done
            self._mark(f"own columns {p} split", lib)
            self._record(self._ev_planes[R][p], lib)

        ahead = self.ahead
        # the first two panels' shares are split before this rank's rows of A are: their exchange
        # then runs beside the preparation of A instead of behind it
        prepared = pulled = 0
        while prepared < min(2, P):
            stage_prep(prepared)
            prepared += 1
        if self.rows:
            self.backend.begin(A_rows, max(wd for _, wd in self.cols))
            self._mark("A prepared", lib)
        arrived = [None] * P

        def pull_planes(p: int) -> None:
            for i in range(1, W):
                q = (R + i) % W
                if not self._regions[p][q]:
                    continue
                st = pool[i % len(pool)]
                self._wait(self._ev_planes[q][p], st)
                self._mark(f"planes {p} of rank {q} ready", st)
                for off, width, rows, pitch in self._regions[p][q]:
                    self._copy2d(self._blk_P[p].ptr + off, pitch, self._addr_P[q][p] + off, pitch, width, rows, st)
                self._mark(f"planes {p} of rank {q} here", st)
            for st in pool:
                x2.wait_stream(st)
            arrived[p] = torch.cuda.Event()
            arrived[p].record(x2)
            self._mark(f"planes {p} arrived", x2)

        for p in range(P):
            # every rank has called the records so far (the planes of the panels staged up to
            # here, the block of panel p - 1) before any peer calls their waits
            self._host_mark(f"iteration {p}")
            dist.barrier(group=self.ctl)
            self._host_mark(f"barrier {p} passed")
            c0p, wd = self.cols[p]
            # the planes of every panel staged so far are on their way: `ahead` panels beyond the
            # one being multiplied (two is the measured optimum on 8 GPUs: with three or four in
            # flight the step was slower there)
            while pulled < prepared:
                pull_planes(pulled)
                pulled += 1
            self._host_mark(f"pulls of {p} called")
            if self.rows:
                lib.wait_event(arrived[p])
                self._mark(f"panel {p} products start", lib)
                if lib_h.eshkol_b200_adopt_prepared_b(self._blk_P[p].ptr, self.K, wd) != 0:
                    raise RuntimeError("adopt_prepared_b failed")
                c = self.C[self.row0:self.row0 + self.rows, c0p:c0p + wd]
                opts = self.backend.api.make_opts(self.backend.tier, self.backend.param, ldc=c.stride(0))
                if lib_h.eshkol_b200_multiply_prepared_f64_device(c.data_ptr(), ctypes.byref(opts)) != 0:
                    raise RuntimeError("multiply failed")
                self._mark(f"panel {p} products done", lib)
            self._record(self._ev_block[R][p], lib)
            self._host_mark(f"products {p} called")
            # behind the products of panel p: the shares of the panels up to p + ahead
            while prepared < P and prepared <= p + ahead:
                stage_prep(prepared)
                prepared += 1
            # the blocks of C of the panel before this one, on streams of their own: every rank
            # has called their records (they precede this iteration's barrier)
            self._host_mark(f"stages after {p} called")
            if p >= 1:
                self._gather_panel(p - 1, gpool, xo)
        self._host_mark("loop done")
        dist.barrier(group=self.ctl)
        self._gather_panel(P - 1, gpool, xo)
        cur.wait_stream(lib)
        cur.wait_stream(xo)
        cur.wait_stream(x1)
        cur.wait_stream(x2)
        self.backend.finish()
        cur.synchronize()
        dist.barrier(group=self.ctl)  # nobody overwrites a buffer a peer may still be reading
        return self.C

    def _gather_panel(self, p: int, pool, xo) -> None:
        """pull every other rank's block of panel p of C into its place, once it is computed"""
        R, W = self.rank, self.world
        for i in range(1, W):
            q = (R + i) % W
            if self.parts[q][1] == 0:
                continue
            st = pool[i % len(pool)]
            self._wait(self._ev_block[q][p], st)
            self._mark(f"block {p} of rank {q} ready", st)
            self._pull_c_block(q, p, st)
            self._mark(f"block {p} of rank {q} here", st)
        for st in pool:
            xo.wait_stream(st)
        self._mark(f"panel {p} gathered", xo)

    def _unpack(self, p: int) -> None:
        """gathered panel p, [rank][row][column in panel] -> its columns of the row-major C"""
        w = self.width
        dst = self.C[:, p * w:(p + 1) * w]
        if self.world * self.max_rows == self.M:
            dst.copy_(self.Cp[p].view(self.M, w))
        else:
            for r, (r0, rows) in enumerate(self.parts):
                dst[r0:r0 + rows].copy_(self.Cp[p, r, :rows])

    def _host_mark(self, label: str) -> None:
        """host time of a point of the traced step (beside the device marks of _mark)"""
        if self.trace is not None:
            import time
            self.host_trace.append((label, time.perf_counter()))

    def _mark(self, label: str, stream) -> None:
        if self.trace is not None and stream is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            self.trace.append((label, ev))

    def trace_ms(self) -> list[tuple[str, float]]:
        """Marks of the traced step as milliseconds after its first mark (call after the step)."""
        if not self.trace:
            return []
        t0 = self.trace[0][1]
        return [(label, t0.elapsed_time(ev)) for label, ev in self.trace]

    def step(self, A_rows: torch.Tensor, B_src: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One product.  A_rows: this rank's rows (rows x K).  B_src: the full B on rank `src`.
        Returns the full C (M x N), identical on every rank.

        On GPUs the whole step is enqueued without a host wait: the packing of a panel, its
        broadcast, the library's kernels, the gather of the panel's block of C and its unpacking
        into C are ordered by stream events, so the broadcast of panel p+1, the products of
        panel p, the gather of panel p-1 and the unpacking of panel p-2 run at the same time.
        One host wait at the end reads the kernels' status word."""
        if A_rows.shape != (self.rows, self.K):
            raise ValueError(f"rank {self.rank} expects {self.rows} x {self.K} rows of A")
        P, w = self.panels, self.width
        dev = self.backend.on_device
        cur = torch.cuda.current_stream(self.device) if dev else None
        lib = self.backend.stream if dev else None
        if dev and self._side is None:
            self._side = torch.cuda.Stream(self.device)
        side = self._side
        if self.rank == self.src and B_src is None:
            raise ValueError("the source rank must pass B")
        if self.transport == "copy_engine":
            if self.split_shared:
                return self._step_shared_split(A_rows, B_src)
            return self._step_copy_engine(A_rows, B_src)
        self._mark("start", cur)
        if dev:
            side.wait_stream(cur)  # whoever read C after the last step did so on torch's stream
        if self.rows:
            if dev:
                lib.wait_stream(cur)  # A was produced on torch's stream
            self.backend.begin(A_rows, w)
            self._mark("A prepared", lib)
        arrivals = []
        for p in range(P):
            if self.rank == self.src:
                self.Bp[p].copy_(B_src[:, p * w:(p + 1) * w])
            if self.world > 1:
                arrivals.append(dist.broadcast(self.Bp[p], src=self.src, group=self.group, async_op=True))
        gathers = []
        for p in range(P):
            if arrivals:
                arrivals[p].wait()  # orders torch's stream (on CPU: the host) behind the broadcast
                self._mark(f"B panel {p} arrived", cur)
            if self.rows:
                if dev:
                    lib.wait_stream(cur)
                self._mark(f"panel {p} products start", lib)
                self.backend.panel(A_rows, self.Bp[p], self.Cp[p, self.rank, : self.rows])
                self._mark(f"panel {p} products done", lib)
                if dev:
                    cur.wait_stream(lib)
            if self.world > 1:
                gathers.append(dist.all_gather_into_tensor(
                    self.Cp[p].view(self.world * self.max_rows, w), self.Cp[p, self.rank],
                    group=self.group, async_op=True))
            # the panel before this one has had a whole panel's products to arrive: unpack it
            # beside the products now running
            q = p - 1
            if q >= 0:
                if dev:
                    with torch.cuda.stream(side):
                        if gathers:
                            gathers[q].wait()
                        else:
                            side.wait_stream(cur)
                        self._mark(f"panel {q} gathered", side)
                        self._unpack(q)
                else:
                    if gathers:
                        gathers[q].wait()
                    self._unpack(q)
        if dev:
            with torch.cuda.stream(side):
                if gathers:
                    gathers[P - 1].wait()
                else:
                    side.wait_stream(cur)
                self._mark(f"panel {P - 1} gathered", side)
                self._unpack(P - 1)
                self._mark("unpacked", side)
            cur.wait_stream(side)
        else:
            if gathers:
                gathers[P - 1].wait()
            self._unpack(P - 1)
        self.backend.finish()
        if dev:
            cur.synchronize()
        return self.C

    def result(self) -> torch.Tensor:
        return self.C
