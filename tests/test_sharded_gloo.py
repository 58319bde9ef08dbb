"""world_size-2 (and 3) gloo runs of the row-sharded path on CPU.

The device kernel is replaced by the CPU oracle through `local_gemm`, so what is
exercised is the host logic that has to be right on N GPUs: the row ranges, the
byte offsets of a shard, the all-gather and the re-assembly of [M x N]."""
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
from oxillama_b200 import synth as S  # noqa: E402
from oxillama_b200.sharded import RowShardedLinear, row_bytes, shard_rows  # noqa: E402


def _worker(rank, world, port, qtype, rows, cols, m, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = S.gen_weight(qtype, rows, cols, seed=41)
        x = S.gen_acts(m, cols, seed=41)
        b, e = shard_rows(rows, world, rank)
        rb = row_bytes(qtype, cols)

        def local_gemm(xt, yt, mm):
            st, y = O.gemm(qtype, w[b * rb: e * rb], xt.numpy(), mm, e - b, cols)
            assert st == 0
            yt.copy_(torch.from_numpy(y))

        lin = RowShardedLinear(qtype, w, rows, cols, local_gemm=local_gemm, device=torch.device("cpu"))
        assert (lin.begin, lin.end) == (b, e)
        y = lin.forward(torch.from_numpy(x), m).numpy()
        st, ref = O.gemm(qtype, w, x, m, rows, cols)
        assert st == 0
        out[rank] = bool(np.array_equal(y, ref))  # same oracle rows on every rank: exact
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,qtype,rows,cols,m", [
    (2, S.Q4_K, 64, 512, 1), (2, S.Q4_K, 64, 512, 3), (2, S.Q6_K, 37, 256, 2), (3, S.Q8_0, 40, 96, 4)])
def test_row_sharded_equals_single(world, qtype, rows, cols, m):
    port = 29500 + (os.getpid() + world * 7 + rows) % 2000
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, qtype, rows, cols, m, out), nprocs=world, join=True)
        assert all(out.get(r) for r in range(world)), dict(out)


def test_shard_rows_partition():
    for n in (0, 1, 7, 8, 4096, 128256):
        for g in (1, 2, 3, 4, 8):
            spans = [shard_rows(n, g, r) for r in range(g)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(g - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
