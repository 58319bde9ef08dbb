"""Expert sharding of the MoE layer: host-side logic on CPU ranks (gloo, world size 2).

Each rank computes its experts' contribution with a numpy stand-in for the
device call, the ranks' outputs are summed with a gloo all-reduce, and the
result must equal the oracle's whole-layer output
(crates/oxillama-arch/src/common/moe.rs:184-258).  The token exchange (every rank owns
its own tokens, routed rows cross by all-to-all) runs the same way, with numpy stand-ins
for the device calls and gloo's all-to-all.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import oracle_lib as O  # noqa: E402
from oxillama_b200 import moe  # noqa: E402


def test_expert_range_partitions():
    for n, w in ((8, 1), (8, 2), (8, 8), (8, 3), (5, 4), (2, 4)):
        got = [moe.expert_range(n, w, r) for r in range(w)]
        assert got[0][0] == 0 and got[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
        sizes = [e - b for b, e in got]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        moe.expert_range(8, 2, 2)


def _local_numpy(gate, up, down, begin, end):
    """Contribution of experts [begin, end) in plain numpy f32, routed by the oracle."""
    def fwd(logits, x, top_k):
        lg, xn = logits.numpy(), x.numpy()
        ids, wts = O.moe_route(lg, top_k)
        y = np.zeros_like(xn)
        for t in range(xn.shape[0]):
            for k in range(top_k):
                e = int(ids[t, k])
                if begin <= e < end:
                    g = gate[e] @ xn[t]
                    h = (g / (1.0 + np.exp(-g))) * (up[e] @ xn[t])
                    y[t] += wts[t, k] * (down[e] @ h)
        return torch.from_numpy(y.astype(np.float32))
    return fwd


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(9)
    n_exp, hidden, inter, tokens, top_k = 4, 32, 48, 12, 2
    gate = rng.standard_normal((n_exp, inter, hidden)).astype(np.float32) * 0.2
    up = rng.standard_normal((n_exp, inter, hidden)).astype(np.float32) * 0.2
    down = rng.standard_normal((n_exp, hidden, inter)).astype(np.float32) * 0.2
    logits = rng.standard_normal((tokens, n_exp)).astype(np.float32)
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    b, e = moe.expert_range(n_exp, world, rank)
    layer = moe.ExpertShardedMoe(n_exp, world, rank, _local_numpy(gate, up, down, b, e))
    y = layer.forward(torch.from_numpy(logits), torch.from_numpy(x), top_k).numpy()
    ref = O.moe_ffn_f32(gate, up, down, logits, x, top_k)
    q.put((rank, float(np.abs(y - ref).max() / np.abs(ref).max())))
    dist.destroy_process_group()


def test_expert_sharded_moe_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(err <= 1e-5 for _, err in res), res


def test_exchange_plan():
    ids = np.array([[0, 3], [2, 3], [1, 0], [-1, -1], [3, 1]], dtype=np.int32)
    send_idx, counts, back = moe.exchange_plan(ids, 4, 2)  # experts 0, 1 on rank 0; 2, 3 on rank 1
    assert send_idx.tolist() == [0, 2, 4, 0, 1, 4] and counts.tolist() == [3, 3]
    assert back.tolist() == [[0, 3], [4, -1], [1, -1], [-1, -1], [2, 5]]
    send_idx, counts, back = moe.exchange_plan(np.empty((0, 2), np.int32), 4, 2)
    assert len(send_idx) == 0 and counts.tolist() == [0, 0] and back.shape == (0, 2)
    # more ranks than slots: a token has at most top_k rows out
    send_idx, counts, back = moe.exchange_plan(np.array([[5, 0]], dtype=np.int32), 8, 8)
    assert counts.tolist() == [1, 0, 0, 0, 0, 1, 0, 0] and back.tolist() == [[0, 1]]
    assert moe.expert_owner(5, 4).tolist() == [0, 0, 1, 2, 3]


def test_exchange_plan_properties():
    """Random routings: every (token, owning rank) pair is sent exactly once, in rank-major token
    order; the counts match; the return table names each token's rows in rank order."""
    rng = np.random.default_rng(21)
    for n_exp, world, top_k, tokens in ((8, 8, 2, 33), (8, 2, 2, 17), (5, 4, 3, 9), (4, 1, 2, 6), (16, 8, 4, 64)):
        ids = np.stack([rng.permutation(n_exp)[:top_k] for _ in range(tokens)]).astype(np.int32)
        ids[rng.integers(0, tokens), top_k - 1] = -1  # an empty slot
        owner = moe.expert_owner(n_exp, world)
        send_idx, counts, back = moe.exchange_plan(ids, n_exp, world)
        want = sorted({(int(owner[e]), t) for t in range(tokens) for e in ids[t] if e >= 0})
        ranks = np.repeat(np.arange(world), counts)
        assert list(zip(ranks.tolist(), send_idx.tolist())) == want
        assert back.shape == (tokens, max(1, min(top_k, world)))
        for t in range(tokens):
            rows = [j for j in back[t].tolist() if j >= 0]
            assert [(int(ranks[j]), int(send_idx[j])) for j in rows] == [p for p in want if p[1] == t]
            assert all(j == -1 for j in back[t, len(rows):].tolist())


def _cpu_hooks():
    """numpy / torch-on-CPU stand-ins for the device entry points of the token exchange."""
    def route_ids(logits, top_k):
        return torch.from_numpy(O.moe_route(logits.numpy(), top_k)[0].astype(np.int32))

    def take(x, idx):
        return x[idx.long()].contiguous()

    def total(src, table, width):
        y = torch.zeros((table.shape[0], width), dtype=torch.float32)
        for t in range(table.shape[0]):
            for j in table[t].tolist():
                if j >= 0:
                    y[t] += src[j]
        return y
    return dict(route_ids=route_ids, take=take, total=total)


def _exchange_worker(rank, world, port, q, cuts, n_exp=4):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(11)
    hidden, inter, tokens, top_k = 32, 48, 12, 2
    gate = rng.standard_normal((n_exp, inter, hidden)).astype(np.float32) * 0.2
    up = rng.standard_normal((n_exp, inter, hidden)).astype(np.float32) * 0.2
    down = rng.standard_normal((n_exp, hidden, inter)).astype(np.float32) * 0.2
    logits = rng.standard_normal((tokens, n_exp)).astype(np.float32)
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    b, e = moe.expert_range(n_exp, world, rank)
    lo, hi = cuts[rank], cuts[rank + 1]  # this rank's own tokens
    layer = moe.TokenExchangeMoe(n_exp, world, rank, _local_numpy(gate, up, down, b, e), **_cpu_hooks())
    y = layer.forward(torch.from_numpy(logits[lo:hi].copy()), torch.from_numpy(x[lo:hi].copy()), top_k).numpy()
    ref = O.moe_ffn_f32(gate, up, down, logits, x, top_k)[lo:hi]
    err = float(np.abs(y - ref).max() / np.abs(ref).max()) if hi > lo else 0.0
    q.put((rank, y.shape == ref.shape, err))
    dist.destroy_process_group()


# ragged shares; a rank without tokens, either one; three ranks with 2, 2 and 1 of five experts
@pytest.mark.parametrize("cuts,n_exp", [((0, 7, 12), 4), ((0, 0, 12), 4), ((0, 12, 12), 4), ((0, 5, 5, 12), 5)])
def test_token_exchange_moe_ranks(cuts, n_exp):
    world = len(cuts) - 1
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000) + cuts[1] + 16 * world
    procs = [ctx.Process(target=_exchange_worker, args=(r, world, port, q, cuts, n_exp)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _, _ in res) == list(range(world))
    assert all(ok and err <= 1e-5 for _, ok, err in res), res
