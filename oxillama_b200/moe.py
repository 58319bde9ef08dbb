"""Mixture-of-experts FFN over device-resident quantized experts.

Mirrors `MoeFfn::forward` / `Expert::forward` of the reference
(crates/oxillama-arch/src/common/moe.rs:184-258, 75-126): router logits ->
softmax -> top-k -> renormalised weights -> sum of the selected experts'
`down(silu(gate x) * up x)`.  The arithmetic runs in libqk_cuda.so
(`qk_moe_ffn_dev`); this module only holds handles and torch buffers.

Expert sharding (one process per GPU): every rank holds a contiguous range of
experts, computes their contribution for all tokens, and the ranks' outputs are
summed (`ExpertShardedMoe`).
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Sequence

import numpy as np

from . import synth as S


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [begin, end) of `rank`: as even as possible, earlier ranks take the remainder."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, rem = divmod(n_experts, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class MoeExperts:
    """gate / up / down of a contiguous range of experts, resident on one GPU."""

    def __init__(self, tensor_type: int, gate: Sequence[np.ndarray], up: Sequence[np.ndarray],
                 down: Sequence[np.ndarray], hidden: int, inter: int, n_experts: int, expert_begin: int = 0,
                 ctx=None):
        from .device import DeviceWeights
        from .kernels import default_context
        if not (len(gate) == len(up) == len(down)):
            raise ValueError("gate, up and down need one matrix per local expert")
        if expert_begin + len(gate) > n_experts:
            raise ValueError("local experts exceed the expert count")
        self.ctx = ctx or default_context()
        self.hidden, self.inter, self.n_experts, self.expert_begin = hidden, inter, n_experts, expert_begin
        self.gate = [DeviceWeights(tensor_type, w, inter, hidden, ctx=self.ctx) for w in gate]
        self.up = [DeviceWeights(tensor_type, w, inter, hidden, ctx=self.ctx) for w in up]
        self.down = [DeviceWeights(tensor_type, w, hidden, inter, ctx=self.ctx) for w in down]
        n = len(gate)
        arr = C.c_void_p * max(n, 1)
        self._g = arr(*[d.handle for d in self.gate])
        self._u = arr(*[d.handle for d in self.up])
        self._d = arr(*[d.handle for d in self.down])

    @property
    def n_local(self) -> int:
        return len(self.gate)

    def forward(self, logits, x, y, top_k: int, stream=None) -> None:
        """y[tokens x hidden] = contribution of the local experts (overwrites y)."""
        import torch
        from .device import _stream_ptr
        tokens = x.shape[0]
        for t, shape, what in ((logits, (tokens, self.n_experts), "logits"), (x, (tokens, self.hidden), "x"),
                               (y, (tokens, self.hidden), "y")):
            if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == shape):
                raise TypeError(f"{what}: need a contiguous CUDA float32 tensor of shape {shape}")
        self.ctx.check(self.ctx.lib.qk_moe_ffn_dev(
            self.ctx.handle, self._g, self._u, self._d, self.n_local, self.expert_begin, self.n_experts,
            C.c_void_p(logits.data_ptr()), C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), tokens, top_k,
            _stream_ptr(stream)))

    def free(self):
        for d in self.gate + self.up + self.down:
            d.free()


def route(logits, top_k: int, ctx=None, stream=None):
    """(ids int32 [tokens x top_k], weights f32 [tokens x top_k]) of `qk_moe_route_dev`."""
    import torch
    from .device import _stream_ptr
    from .kernels import default_context
    ctx = ctx or default_context()
    tokens, n_exp = logits.shape
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((tokens, top_k), dtype=torch.float32, device=logits.device)
    ctx.check(ctx.lib.qk_moe_route_dev(ctx.handle, C.c_void_p(logits.data_ptr()), tokens, n_exp, top_k,
                                       C.c_void_p(ids.data_ptr()), C.c_void_p(wts.data_ptr()), _stream_ptr(stream)))
    return ids, wts


class ExpertShardedMoe:
    """One rank of an expert-sharded MoE layer.

    `local_forward(logits, x, top_k) -> y_local` computes this rank's experts'
    contribution (on a GPU: `MoeExperts.forward`); `all_reduce_sum(y)` sums it
    over the ranks in place (NCCL on GPUs, gloo in the CPU tests).
    """

    def __init__(self, n_experts: int, world: int, rank: int, local_forward: Callable,
                 all_reduce_sum: Callable | None = None):
        self.begin, self.end = expert_range(n_experts, world, rank)
        self.world, self.rank = world, rank
        self.local_forward, self.all_reduce_sum = local_forward, all_reduce_sum

    def forward(self, logits, x, top_k: int):
        y = self.local_forward(logits, x, top_k)
        if self.world > 1:
            if self.all_reduce_sum is None:
                import torch.distributed as dist
                dist.all_reduce(y)
            else:
                self.all_reduce_sum(y)
        return y
