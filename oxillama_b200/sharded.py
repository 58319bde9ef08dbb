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


class _DevPtr:
    """Lets torch view device memory owned by libqk_cuda.so (`__cuda_array_interface__`)."""

    def __init__(self, ptr: int, shape, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 2}


class PeerGather:
    """Gathered outputs of a row-sharded layer over the GPUs of one node, without a
    collective: every rank's matvec stores its block, as (value, tag) words, into a slot
    array of every rank over NVLink (`qk_gemm_gather_dev`); the consumer is either the next
    sharded matvec, which reads its activations straight from the slots as they arrive
    (`after=`), or `wait()`, which unpacks them into `buffer`.  Every wait is bounded.  The
    ranks exchange the CUDA IPC handles of their slot arrays through `torch.distributed`
    (any host channel would do).

    Every rank must issue the same sequence of calls on a `PeerGather`.  A call overwrites
    the previous call's slots in every rank: alternate two objects when each call waits for
    the one before it, four when the wait trails by one call.
    """

    def __init__(self, rows_per_rank: int, m_cap: int = 1, group: Optional[dist.ProcessGroup] = None, ctx=None,
                 _local=None):
        import ctypes as C
        from .kernels import default_context
        self.ctx = ctx or default_context()
        self.group = group
        self.rows, self.m_cap = rows_per_rank, m_cap
        self._siblings = None
        if _local is not None:  # one of several ranks emulated inside this process (see local_world)
            self.world, self.rank = _local
            h = C.c_void_p()
            self.ctx.check(self.ctx.lib.qk_gather_create(self.ctx.handle, rows_per_rank, m_cap, self.world,
                                                         self.rank, C.byref(h)))
            self.handle = h
            self._view()
            return
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # Failures are agreed on by all ranks before anyone raises, so that no rank is left
        # waiting in a collective for one that has already given up.
        h, err, payload = C.c_void_p(), None, None
        try:
            self.ctx.check(self.ctx.lib.qk_gather_create(self.ctx.handle, rows_per_rank, m_cap, self.world,
                                                         self.rank, C.byref(h)))
            if self.world > 1:
                buf = (C.c_ubyte * 128)()
                self.ctx.check(self.ctx.lib.qk_gather_export(self.ctx.handle, h, buf, 128))
                payload = bytes(buf)
        except Exception as e:  # noqa: BLE001
            err = e
        self.handle = h if err is None else None
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, payload, group=group)
            if err is None and all(hb is not None for hb in handles):
                try:
                    for r, hb in enumerate(handles):
                        if r != self.rank:
                            pb = (C.c_ubyte * 128).from_buffer_copy(hb)
                            self.ctx.check(self.ctx.lib.qk_gather_import(self.ctx.handle, h, r, pb, 128))
                    self.ctx.check(self.ctx.lib.qk_gather_ready(self.ctx.handle, h))
                except Exception as e:  # noqa: BLE001
                    err = e
            elif err is None:
                err = RuntimeError("a peer rank could not create or export its gather buffer")
            oks = [None] * self.world
            dist.all_gather_object(oks, err is None, group=group)
            if err is None and not all(oks):
                err = RuntimeError("a peer rank could not import the gather buffers")
        if err is not None:  # every rank is here (the failure was agreed on above)
            if h:
                self.ctx.lib.qk_gather_close_peers(self.ctx.handle, h)
            if self.world > 1:
                dist.barrier(group=group)
            if h:
                self.ctx.lib.qk_gather_destroy(self.ctx.handle, h)
            self.handle = None
            raise err
        self._view()

    @classmethod
    def local_world(cls, rows_per_rank: int, world: int, m_cap: int = 1, ctx=None) -> "list[PeerGather]":
        """`world` ranks inside this process and on this GPU, wired to one another without IPC:
        what a single-GPU test drives to exercise the cross-rank protocol (the ranks' calls
        are enqueued one after another on one stream, producers before their consumers)."""
        ranks = [cls(rows_per_rank, m_cap, ctx=ctx, _local=(world, r)) for r in range(world)]
        for a in ranks:
            for b in ranks:
                if a is not b:
                    a.ctx.check(a.ctx.lib.qk_gather_import_local(a.ctx.handle, a.handle, b.rank, b.handle))
        for a in ranks:
            a.ctx.check(a.ctx.lib.qk_gather_ready(a.ctx.handle, a.handle))
            a._siblings = ranks
        return ranks

    def _view(self):
        ptr = self.ctx.lib.qk_gather_buffer(self.handle)
        self.buffer = torch.as_tensor(_DevPtr(ptr, (self.m_cap, self.world * self.rows)), device="cuda")

    def gemm(self, dw, x: torch.Tensor, m: int = 1, after: "PeerGather | None" = None,
             unpack: "PeerGather | None" = None, stream=None) -> None:
        """Enqueues this rank's shard matvec with its result fanned out to every rank.

        `after`: x lies inside `after.buffer` and stands for the gathered output of the latest
        call on that PeerGather; the kernels read it from the arriving slots (or unpack it
        first where they cannot).  `unpack`: the latest call on that other PeerGather is
        unpacked into its `buffer` in passing (what `unpack.wait()` does, without a kernel of
        its own where the matvec kernel can do it)."""
        import ctypes as C
        from .device import _stream_ptr
        self.ctx.check(self.ctx.lib.qk_gemm_gather_unpack_dev(
            self.ctx.handle, dw.handle, C.c_void_p(x.data_ptr()), m, self.handle,
            after.handle if after is not None else None, unpack.handle if unpack is not None else None,
            _stream_ptr(stream)))

    def wait(self, stream=None) -> None:
        """Enqueues the (bounded) wait for every block of the latest call; `buffer` then holds it."""
        from .device import _stream_ptr
        self.ctx.check(self.ctx.lib.qk_gather_wait_dev(self.ctx.handle, self.handle, _stream_ptr(stream)))

    def _teardown(self, h):
        # two steps with a rendezvous between them: nobody frees arrays a peer still has open
        self.ctx.lib.qk_gather_close_peers(self.ctx.handle, h)
        if self.world > 1 and self._siblings is None and dist.is_initialized():
            dist.barrier(group=self.group)
        self.ctx.lib.qk_gather_destroy(self.ctx.handle, h)

    def free(self):
        if self.handle:
            self.buffer = None
            if self._siblings is not None:  # in-process ranks: close every rank's view first
                torch.cuda.synchronize()
                for sib in self._siblings:
                    if sib.handle:
                        sib.ctx.lib.qk_gather_close_peers(sib.ctx.handle, sib.handle)
            elif self.world > 1:
                torch.cuda.synchronize()
                dist.barrier(group=self.group)  # nobody may still be storing into this rank's slots
            self._teardown(self.handle)
            self.handle = None
