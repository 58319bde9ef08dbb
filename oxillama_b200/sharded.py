"""Row-sharded linear layers over several GPUs (one process per GPU).

The reference has no multi-device path; its `QuantLinear::forward` /
`forward_batch` (crates/oxillama-arch/src/common/linear.rs:77-132) compute
y = W x on one host.  Rows of W are independent dot products and a row range is
a contiguous byte range of the GGUF tensor, so rank g of G keeps rows
[g*N/G, (g+1)*N/G) resident, computes its slice of y, and one all-gather over
the process group (NCCL over NVLink on GPUs, gloo in the CPU tests) rebuilds
the full output on every rank.  Parity statement: the gathered result equals the
single-device result, which equals the oracle.

torch.distributed is plumbing here; the arithmetic is the `local_gemm`
callable, by default the CUDA library through `DeviceWeights`.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch
import torch.distributed as dist

from .synth import BLOCK_BYTES, BLOCK_SIZE


def shard_rows(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [begin, end) owned by `rank`: contiguous, sizes differ by at most one."""
    base, rem = divmod(n_rows, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def row_bytes(tensor_type: int, n_cols: int) -> int:
    bs = BLOCK_SIZE[tensor_type]
    return -(-n_cols // bs) * BLOCK_BYTES[tensor_type]


class RowShardedLinear:
    """y[m, :] = W x[m, :] with W row-sharded across the ranks of `group`.

    `local_gemm(x, y_local, m)` must fill y_local[m, rows_local] from x[m, n_cols]
    for this rank's rows; when omitted the rows are uploaded to the current CUDA
    device and `DeviceWeights.gemm` is used.
    """

    def __init__(self, tensor_type: int, data: np.ndarray, n_rows: int, n_cols: int,
                 group: Optional[dist.ProcessGroup] = None,
                 local_gemm: Optional[Callable] = None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.tensor_type, self.n_rows, self.n_cols = tensor_type, n_rows, n_cols
        self.begin, self.end = shard_rows(n_rows, self.world, self.rank)
        self.rows_local = self.end - self.begin
        self.max_local = shard_rows(n_rows, self.world, 0)[1]  # rank 0 holds the largest shard
        self.device = device
        self._dw = None
        if local_gemm is None:
            from .device import DeviceWeights
            self._dw = DeviceWeights(tensor_type, data, n_rows, n_cols, self.begin, self.end)
            self.device = torch.device("cuda", torch.cuda.current_device())

            def local_gemm(x, y_local, m):
                self._dw.gemm(x, y_local, m)
        self.local_gemm = local_gemm
        self.algo_bytes = self.rows_local * row_bytes(tensor_type, n_cols)

    def forward(self, x: torch.Tensor, m: int = 1) -> torch.Tensor:
        """x: [m, n_cols] f32 on this rank's device -> y: [m, n_rows] on every rank."""
        dev = self.device or x.device
        y_local = torch.empty((m, self.max_local), dtype=torch.float32, device=dev)
        if self.rows_local < self.max_local:
            y_local.zero_()
        if self.rows_local:
            tight = y_local if self.rows_local == self.max_local else \
                torch.empty((m, self.rows_local), dtype=torch.float32, device=dev)
            self.local_gemm(x, tight, m)
            if tight is not y_local:
                y_local[:, : self.rows_local] = tight
        if self.world == 1:
            return y_local[:, : self.n_rows]
        gathered = torch.empty((self.world * m, self.max_local), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(gathered, y_local, group=self.group)  # rank-major concatenation
        return assemble(gathered.view(self.world, m, self.max_local), self.n_rows, self.world)

    def free(self):
        if self._dw is not None:
            self._dw.free()
            self._dw = None


def assemble(gathered: torch.Tensor, n_rows: int, world: int) -> torch.Tensor:
    """[world, m, max_local] rank-major slices -> [m, n_rows] row-major output."""
    m = gathered.shape[1]
    if m == 1 and n_rows % world == 0:
        return gathered.reshape(1, n_rows)  # already contiguous in the right order
    parts = []
    for r in range(world):
        b, e = shard_rows(n_rows, world, r)
        parts.append(gathered[r, :, : e - b])
    return torch.cat(parts, dim=1)
