"""Mixture-of-experts FFN over device-resident quantized experts.

Mirrors `MoeFfn::forward` / `Expert::forward` of the reference
(crates/oxillama-arch/src/common/moe.rs:184-258, 75-126): router logits ->
softmax -> top-k -> renormalised weights -> sum of the selected experts'
`down(silu(gate x) * up x)`.  The arithmetic runs in libqk_cuda.so
(`qk_moe_ffn_dev`); this module only holds handles and torch buffers.

Expert sharding (one process per GPU): every rank holds a contiguous range of
experts, computes their contribution for all tokens, and the ranks' outputs are
summed (`ExpertShardedMoe`).  Where every rank owns its own tokens instead, only the
routed rows cross between the ranks, by two all-to-all exchanges (`TokenExchangeMoe`).
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


def expert_owner(n_experts: int, world: int):
    """owner[e] = the rank whose `expert_range` holds expert e."""
    owner = np.empty(n_experts, dtype=np.int64)
    for r in range(world):
        b, e = expert_range(n_experts, world, r)
        owner[b:e] = r
    return owner


def exchange_plan(ids: np.ndarray, n_experts: int, world: int):
    """Which of this rank's token rows go to which rank, from the routed ids [tokens x top_k].

    A token goes once to every rank that holds at least one of its selected experts (ids
    below zero are empty slots).  Returns `(send_idx, send_counts, back)`: the token
    indices in send order (by rank, then by token), the number of rows per destination
    rank, and an int32 table [tokens x min(top_k, world)] holding, for each token, the
    positions in send order of its rows in rank order, -1 where it has fewer.
    """
    tokens, top_k = ids.shape
    owner = expert_owner(n_experts, world)
    goes = np.zeros((tokens, world), dtype=bool)
    for k in range(top_k):
        sel = ids[:, k] >= 0
        goes[np.nonzero(sel)[0], owner[ids[sel, k]]] = True
    send_counts = goes.sum(axis=0).astype(np.int64)
    ranks, toks = np.nonzero(goes.T)  # rank-major, tokens ascending inside a rank
    send_idx = toks.astype(np.int32)
    per_row = max(1, min(top_k, world))
    back = np.full((tokens, per_row), -1, dtype=np.int32)
    order = np.argsort(toks, kind="stable")  # a token's rows together, still in rank order
    st = toks[order]
    first = np.searchsorted(st, st, side="left")
    back[st, np.arange(len(st)) - first] = order
    return send_idx, send_counts, back


def _need(t, dtype, ndim: int, what: str) -> None:
    if not (t.is_cuda and t.dtype == dtype and t.dim() == ndim and t.is_contiguous()):
        raise TypeError(f"{what}: need a contiguous CUDA tensor of {dtype} with {ndim} dimension(s)")


def take_rows(x, idx, ctx=None, stream=None):
    """x[idx] on the device (`qk_moe_take_rows_dev`): x [n x width] f32, idx int32 [m]."""
    import torch
    from .device import _stream_ptr
    from .kernels import default_context
    ctx = ctx or default_context()
    _need(x, torch.float32, 2, "x")
    _need(idx, torch.int32, 1, "idx")
    out = torch.empty((idx.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
    ctx.check(ctx.lib.qk_moe_take_rows_dev(ctx.handle, C.c_void_p(x.data_ptr()), C.c_void_p(idx.data_ptr()),
                                           idx.shape[0], x.shape[1], C.c_void_p(out.data_ptr()), _stream_ptr(stream)))
    return out


def sum_rows(src, table, width: int, ctx=None, stream=None):
    """y[t] = sum in order of src[table[t][j]] over the entries >= 0 (`qk_moe_sum_rows_dev`)."""
    import torch
    from .device import _stream_ptr
    from .kernels import default_context
    ctx = ctx or default_context()
    _need(table, torch.int32, 2, "table")
    if table.shape[0] and table.shape[1]:
        _need(src, torch.float32, 2, "src")
        if src.shape[1] != width:
            raise ValueError("src rows are not `width` wide")
    y = torch.empty((table.shape[0], width), dtype=torch.float32, device=table.device)
    ctx.check(ctx.lib.qk_moe_sum_rows_dev(ctx.handle, C.c_void_p(src.data_ptr()), C.c_void_p(table.data_ptr()),
                                          table.shape[0], table.shape[1], width, C.c_void_p(y.data_ptr()),
                                          _stream_ptr(stream)))
    return y


class TokenExchangeMoe:
    """One rank of an expert-sharded MoE layer whose tokens are sharded as well.

    Every rank owns its own tokens and a contiguous range of experts.  Only routed rows
    cross between the ranks: a token's activation row and its logits row go once to each
    rank that holds one of its selected experts (one all-to-all of packed rows), that rank computes its
    experts' weighted contribution for the rows it received (`local_forward`, on a GPU
    `MoeExperts.forward`: the router is a function of the token's own logits row, so the
    receiver recomputes the same ids and weights), the partial outputs return by the
    reverse all-to-all, and the owner adds a token's partials in rank order.

    The step is split in three so that a test can drive several ranks of one process in
    lock-step: `begin` (route, plan, pack), `compute` (the local experts over the received
    rows) and `finish` (the sum); `forward` runs them around the two exchanges.
    The hooks default to the device entry points and `torch.distributed`:
    `route_ids(logits, top_k) -> int32 [tokens x top_k]`, `take(x, idx)`, `total(src, table, width)`,
    `all_to_all(out, inp, out_counts, in_counts)`.
    """

    def __init__(self, n_experts: int, world: int, rank: int, local_forward: Callable,
                 route_ids: Callable | None = None, take: Callable | None = None, total: Callable | None = None,
                 all_to_all: Callable | None = None):
        self.n_experts, self.world, self.rank = n_experts, world, rank
        self.begin_expert, self.end_expert = expert_range(n_experts, world, rank)
        self.local_forward = local_forward
        self.route_ids = route_ids or (lambda logits, top_k: route(logits, top_k)[0])
        self.take = take or take_rows
        self.total = total or sum_rows
        self.all_to_all = all_to_all or self._dist_all_to_all

    @staticmethod
    def _dist_all_to_all(out, inp, out_counts, in_counts):
        import torch.distributed as dist
        dist.all_to_all_single(out, inp, list(out_counts), list(in_counts))

    def begin(self, logits, x, top_k: int):
        """Routes the local tokens; returns the packed rows to send and the step's state."""
        import torch
        tokens = x.shape[0]
        if tokens:
            ids = self.route_ids(logits, top_k).cpu().numpy()
        else:
            ids = np.empty((0, top_k), dtype=np.int32)
        send_idx, send_counts, back = exchange_plan(ids, self.n_experts, self.world)
        idx = torch.from_numpy(send_idx).to(x.device)
        state = {"tokens": tokens, "width": x.shape[1], "send_counts": [int(c) for c in send_counts],
                 "back": torch.from_numpy(back).to(x.device), "top_k": top_k}
        if len(send_idx):
            return self.take(x, idx), self.take(logits, idx), state
        return x.new_empty((0, x.shape[1])), logits.new_empty((0, logits.shape[1])), state

    def compute(self, recv_logits, recv_x, top_k: int):
        """The local experts' weighted contribution for the rows received, one row each."""
        if recv_x.shape[0] == 0:
            return recv_x.new_empty((0, recv_x.shape[1]))
        return self.local_forward(recv_logits, recv_x, top_k)

    def finish(self, returned, state):
        """y [tokens x hidden]: every token's partial outputs added in rank order."""
        if state["tokens"] == 0:
            return returned.new_empty((0, state["width"]))
        return self.total(returned, state["back"], state["width"])

    def forward(self, logits, x, top_k: int):
        import torch
        send_x, send_l, st = self.begin(logits, x, top_k)
        sc = st["send_counts"]
        cnt_in = torch.tensor(sc, dtype=torch.int64, device=x.device)
        cnt_out = torch.empty_like(cnt_in)
        self.all_to_all(cnt_out, cnt_in, [1] * self.world, [1] * self.world)
        rc = [int(v) for v in cnt_out.cpu().tolist()]
        # one exchange for both: a row travels as its activations followed by its logits
        hidden = x.shape[1]
        packed = torch.cat((send_x, send_l), dim=1)
        recv = x.new_empty((sum(rc), packed.shape[1]))
        self.all_to_all(recv, packed, rc, sc)
        recv_x, recv_l = recv[:, :hidden].contiguous(), recv[:, hidden:].contiguous()
        part = self.compute(recv_l, recv_x, top_k)
        returned = x.new_empty((sum(sc), x.shape[1]))
        self.all_to_all(returned, part, sc, rc)
        return self.finish(returned, st)
