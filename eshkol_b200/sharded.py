"""Row-sharded f64 GEMM across the GPUs of one box (one process per GPU).

Rows of A are independent in every tier: the scale of row i, its residues and
C[i, :] depend on row i, on B and on the global exponent E only (E = 52 whenever
K <= 131071), so a row shard computed alone carries the same bits as the same rows
of the full product.  Rank r owns a contiguous block of rows of A and of C; B is
broadcast from one rank and the blocks of C are all-gathered, both with
torch.distributed (NCCL over NVLink on GPUs, gloo in the CPU tests).  The reference
has no multi-device code; this is the sharding BASELINE's 32768^3 configuration asks for.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def row_partition(M: int, world: int) -> list[tuple[int, int]]:
    """(first row, row count) per rank: contiguous blocks, sizes differing by at most one."""
    base, extra = divmod(M, world)
    out, start = [], 0
    for r in range(world):
        rows = base + (1 if r < extra else 0)
        out.append((start, rows))
        start += rows
    return out


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
        if self.prepared:
            self._check(self.lib.eshkol_b200_prepare_b_f64_device(b.data_ptr(), b.shape[0], b.shape[1]), "prepare_b")
            self._check(self.lib.eshkol_b200_multiply_prepared_f64_device(c.data_ptr(), None), "multiply")
        else:
            self.api.gemm_device(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape[0], a.shape[1], b.shape[1],
                                 self.api.make_opts(self.tier, self.param))

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
    source rank): all broadcasts are enqueued at once, each panel is multiplied as soon
    as it has arrived, and its block of C is all-gathered while the next panel is being
    multiplied, so only the first broadcast and the last gather are exposed.  All
    buffers are allocated once; step() allocates nothing.

    comm_sms: SMs the products kernels leave free for the collectives.  A products CTA fills
    its SM's shared memory, so a collective's kernel launched beside them would otherwise
    wait for the gap between two products kernels on every rank; the process group should be
    created with as many CTAs at most (NCCL_MAX_CTAS).
    """

    def __init__(self, M: int, K: int, N: int, device, *, tier: int = 0, param: int = 0, src: int = 0,
                 group=None, gemm: Optional[Callable] = None, panels: int = 1, comm_sms: int = 0):
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
        self.panels = panels if (panels > 0 and N % panels == 0) else 1
        self.width = N // self.panels
        # panel-major copy of B: panel p is the contiguous K x width block of columns p*width ...
        self.Bp = torch.empty((self.panels, K, self.width), dtype=torch.float64, device=self.device)
        # gathered blocks: [panel][rank][row][column in panel]; padding rows are never read back
        self.Cp = torch.empty((self.panels, self.world, self.max_rows, self.width), dtype=torch.float64,
                              device=self.device)
        self.C = torch.empty((M, N), dtype=torch.float64, device=self.device)

    def _unpack(self, p: int) -> None:
        """gathered panel p, [rank][row][column in panel] -> its columns of the row-major C"""
        w = self.width
        dst = self.C[:, p * w:(p + 1) * w]
        if self.world * self.max_rows == self.M:
            dst.copy_(self.Cp[p].view(self.M, w))
        else:
            for r, (r0, rows) in enumerate(self.parts):
                dst[r0:r0 + rows].copy_(self.Cp[p, r, :rows])

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
