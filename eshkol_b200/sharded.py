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


def _device_gemm(tier: int, param: int):
    from . import api

    def run(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> None:
        # operands were produced on torch's stream; the library runs on its own
        torch.cuda.current_stream(a.device).synchronize()
        api.gemm_device(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape[0], a.shape[1], b.shape[1],
                        api.make_opts(tier, param))
        st = api.sync_status()
        if st != 0:
            raise RuntimeError(f"GEMM kernel status {st}")

    return run


class ShardedGemm:
    """Buffers and schedule of one sharded product C = A @ B with A row-sharded.

    gemm(a_rows, b, c_rows) computes one shard in place; by default it is the
    library's device GEMM.  All buffers are allocated once, so step() allocates nothing.
    """

    def __init__(self, M: int, K: int, N: int, device, *, tier: int = 0, param: int = 0, src: int = 0,
                 group=None, gemm: Optional[Callable] = None):
        self.M, self.K, self.N = M, K, N
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.src = src
        self.parts = row_partition(M, self.world)
        self.row0, self.rows = self.parts[self.rank]
        self.max_rows = max(r for _, r in self.parts)
        self.device = torch.device(device)
        self.gemm = gemm if gemm is not None else _device_gemm(tier, param)
        self.B = torch.empty((K, N), dtype=torch.float64, device=self.device)
        # gather buffer: world blocks of max_rows rows (padding rows are never read back)
        self.C_blocks = torch.empty((self.world, self.max_rows, N), dtype=torch.float64, device=self.device)

    def step(self, A_rows: torch.Tensor, B_src: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One product.  A_rows: this rank's rows (rows x K).  B_src: the full B on rank `src`."""
        if A_rows.shape != (self.rows, self.K):
            raise ValueError(f"rank {self.rank} expects {self.rows} x {self.K} rows of A")
        if self.rank == self.src:
            if B_src is None:
                raise ValueError("the source rank must pass B")
            if B_src.data_ptr() != self.B.data_ptr():
                self.B.copy_(B_src)
        if self.world > 1:
            dist.broadcast(self.B, src=self.src, group=self.group)
        mine = self.C_blocks[self.rank, : self.rows]
        if self.rows:
            self.gemm(A_rows, self.B, mine)
        if self.world > 1:
            dist.all_gather_into_tensor(self.C_blocks.view(self.world * self.max_rows, self.N),
                                        self.C_blocks[self.rank], group=self.group)
        return self.C_blocks

    def result(self) -> torch.Tensor:
        """The full C (M x N), assembled from the gathered blocks."""
        if self.world * self.max_rows == self.M:
            return self.C_blocks.view(self.M, self.N)
        return torch.cat([self.C_blocks[r, :rows] for r, (_, rows) in enumerate(self.parts)], dim=0)
