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
    tier allows it: A once per step, each column panel of B as it arrives."""

    def __init__(self, tier: int, param: int):
        from . import api
        self.api = api
        self.lib = api.load_library()
        self.tier, self.param = tier, param
        self.prepared = tier == 0 and param in (0, 16)

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc})")

    def begin(self, a: torch.Tensor, panel_cols: int) -> None:
        torch.cuda.current_stream(a.device).synchronize()  # A was produced on torch's stream
        if self.prepared:
            self._check(self.lib.eshkol_b200_prepare_a_f64_device(a.data_ptr(), a.shape[0], a.shape[1], panel_cols),
                        "prepare_a")

    def panel(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> None:
        torch.cuda.current_stream(a.device).synchronize()  # the panel was produced by NCCL
        if self.prepared:
            self._check(self.lib.eshkol_b200_prepare_b_f64_device(b.data_ptr(), b.shape[0], b.shape[1]), "prepare_b")
            self._check(self.lib.eshkol_b200_multiply_prepared_f64_device(c.data_ptr(), None), "multiply")
        else:
            self.api.gemm_device(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape[0], a.shape[1], b.shape[1],
                                 self.api.make_opts(self.tier, self.param))
        st = self.api.sync_status()  # C panel complete before NCCL reads it
        if st != 0:
            raise RuntimeError(f"GEMM kernel status {st}")


class _CallableBackend:
    """gemm(a_rows, b_panel, c_panel) supplied by the caller (CPU tests)."""

    def __init__(self, fn: Callable):
        self.fn = fn

    def begin(self, a, panel_cols) -> None:
        pass

    def panel(self, a, b, c) -> None:
        self.fn(a, b, c)


class ShardedGemm:
    """Buffers and schedule of one sharded product C = A @ B with A row-sharded.

    B travels in `panels` column panels (contiguous K x N/panels blocks packed on the
    source rank): all broadcasts are enqueued at once, each panel is multiplied as soon
    as it has arrived, and its block of C is all-gathered while the next panel is being
    multiplied, so only the first broadcast and the last gather are exposed.  All
    buffers are allocated once; step() allocates nothing.
    """

    def __init__(self, M: int, K: int, N: int, device, *, tier: int = 0, param: int = 0, src: int = 0,
                 group=None, gemm: Optional[Callable] = None, panels: int = 1):
        self.M, self.K, self.N = M, K, N
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.src = src
        self.parts = row_partition(M, self.world)
        self.row0, self.rows = self.parts[self.rank]
        self.max_rows = max(r for _, r in self.parts)
        self.device = torch.device(device)
        self.backend = _CallableBackend(gemm) if gemm is not None else _DeviceBackend(tier, param)
        self.panels = panels if (panels > 0 and N % panels == 0) else 1
        self.width = N // self.panels
        # panel-major copy of B: panel p is the contiguous K x width block of columns p*width ...
        self.Bp = torch.empty((self.panels, K, self.width), dtype=torch.float64, device=self.device)
        # gathered blocks: [panel][rank][row][column in panel]; padding rows are never read back
        self.Cp = torch.empty((self.panels, self.world, self.max_rows, self.width), dtype=torch.float64,
                              device=self.device)
        self.C = torch.empty((M, N), dtype=torch.float64, device=self.device)

    def step(self, A_rows: torch.Tensor, B_src: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One product.  A_rows: this rank's rows (rows x K).  B_src: the full B on rank `src`.
        Returns the full C (M x N), identical on every rank."""
        if A_rows.shape != (self.rows, self.K):
            raise ValueError(f"rank {self.rank} expects {self.rows} x {self.K} rows of A")
        P, w = self.panels, self.width
        if self.rank == self.src:
            if B_src is None:
                raise ValueError("the source rank must pass B")
            for p in range(P):
                self.Bp[p].copy_(B_src[:, p * w:(p + 1) * w])
        arrivals = []
        if self.world > 1:
            arrivals = [dist.broadcast(self.Bp[p], src=self.src, group=self.group, async_op=True)
                        for p in range(P)]
        if self.rows:
            self.backend.begin(A_rows, w)
        gathers = []
        for p in range(P):
            if arrivals:
                arrivals[p].wait()
            if self.rows:
                self.backend.panel(A_rows, self.Bp[p], self.Cp[p, self.rank, : self.rows])
            if self.world > 1:
                gathers.append(dist.all_gather_into_tensor(
                    self.Cp[p].view(self.world * self.max_rows, w), self.Cp[p, self.rank],
                    group=self.group, async_op=True))
        for g in gathers:
            g.wait()
        # [panel][rank][row][col] -> row-major M x N
        if self.world * self.max_rows == self.M:
            self.C.view(self.world, self.max_rows, P, w).copy_(self.Cp.permute(1, 2, 0, 3))
        else:
            for r, (r0, rows) in enumerate(self.parts):
                self.C[r0:r0 + rows].view(rows, P, w).copy_(self.Cp[:, r, :rows].permute(1, 0, 2))
        return self.C

    def result(self) -> torch.Tensor:
        return self.C
