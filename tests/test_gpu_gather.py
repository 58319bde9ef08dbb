"""The cross-rank gather protocol of row-sharded layers, exercised on one GPU.

Several "ranks" live in this process and on this GPU (`PeerGather.local_world`), each with
its own row shard and its own slot array, wired to one another as ranks on different GPUs
are (the peers' arrays are reached through plain device pointers instead of IPC mappings).
The ranks' calls are enqueued on one stream, producers before their consumers, so no
kernel ever waits for one that has not been launched.  What runs is the same code that
runs across NVLink: the matvec kernel's tagged stores into every rank's slots, the next
kernel's reads of its activations out of the arriving slots, the unpacking wait, the call
counting over a thousand calls, and the bounded wait that gives up when a rank never
delivers.  Parity statement: every gathered value equals, bit for bit, what one GPU
computes for the whole matrix (rows are independent dot products), which other tests hold
to the oracle.
"""
import numpy as np
import pytest

import oracle_lib as O
from oxillama_b200 import synth as S

pytestmark = pytest.mark.gpu


def _shards(t, w, rows, cols, world):
    from oxillama_b200.device import DeviceWeights
    from oxillama_b200.sharded import shard_rows
    return [DeviceWeights(t, w, rows, cols, *shard_rows(rows, world, r)) for r in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("t,m", [(S.Q4_K, 1), (S.Q4_K, 3), (S.Q6_K, 1), (S.Q8_0, 9), (S.IQ4_XS, 2)])
def test_gathered_result_equals_single_gpu_and_oracle(world, t, m):
    import torch
    from oxillama_b200.device import DeviceWeights, check_device_status
    from oxillama_b200.sharded import PeerGather
    rows, cols = 40 * world, 1024
    w = S.gen_weight(t, rows, cols, seed=91)
    x = S.gen_acts(m, cols, seed=91)
    st, ref = O.gemm(t, w, x, m, rows, cols)
    assert st == 0
    whole = DeviceWeights(t, w, rows, cols)
    xd = torch.from_numpy(x).cuda()
    y1 = torch.empty((m, rows), device="cuda")
    whole.gemm(xd, y1, m)
    shards = _shards(t, w, rows, cols, world)
    ranks = PeerGather.local_world(rows // world, world, m_cap=m)
    for call in range(3):
        f = float(2 ** call)  # powers of two: exact in every step of the decode kernels
        xs = xd * f
        for r in range(world):
            ranks[r].gemm(shards[r], xs, m)
        for r in range(world):
            ranks[r].wait()
        torch.cuda.synchronize()
        for r in range(world):
            got = ranks[r].buffer[:m]
            if m <= 4:   # decode kernels: the shard computes each row exactly as the whole matrix does
                assert torch.equal(got, y1 * f), (r, call)
            err = np.abs(got.cpu().numpy() - ref * f).max() / np.abs(ref).max() / f
            assert err <= (1e-3 if m > 4 else 2e-5), err
    check_device_status()
    for g in ranks:
        g.free()
    for d in shards + [whole]:
        d.free()


def test_decode_chain_over_a_thousand_calls():
    """Eight chained sharded layers, each reading the gathered output of the one before it out
    of the arriving slots (`after=`), two gather objects alternating per rank, repeated 64
    times without a host synchronisation: 1024 sharded calls per rank, every gathered value
    of every call checked for bit equality with the single-GPU chain."""
    import torch
    from oxillama_b200.device import DeviceWeights, check_device_status
    from oxillama_b200.sharded import PeerGather
    world, n, k0, layers, repeats = 2, 256, 512, 8, 64
    ws = [S.gen_weight(S.Q4_K, n, n if l else k0, seed=92, stream=l, d_range=(1e-3, 2e-3)) for l in range(layers)]
    x0 = torch.from_numpy(S.gen_acts(1, k0, seed=92)).cuda()
    whole = [DeviceWeights(S.Q4_K, ws[l], n, n if l else k0) for l in range(layers)]
    want, cur = [], x0
    for l in range(layers):
        y = torch.empty((1, n), device="cuda")
        whole[l].gemm(cur, y, 1)
        want.append(y)
        cur = y
    assert all(bool(torch.isfinite(v).all()) for v in want)
    shards = [_shards(S.Q4_K, ws[l], n, n if l else k0, world) for l in range(layers)]
    gs = [PeerGather.local_world(n // world, world) for _ in range(2)]   # gs[parity][rank]
    keep = torch.empty((repeats, layers, world, n), device="cuda")
    for rep in range(repeats):
        for l in range(layers):
            cur_g, prev_g = gs[l & 1], gs[(l + 1) & 1]
            for r in range(world):
                if l == 0:
                    cur_g[r].gemm(shards[0][r], x0, 1)
                else:
                    cur_g[r].gemm(shards[l][r], prev_g[r].buffer, 1, after=prev_g[r])
            for r in range(world):
                cur_g[r].wait()
                keep[rep, l, r].copy_(cur_g[r].buffer[0])
    torch.cuda.synchronize()
    check_device_status()
    for l in range(layers):
        assert bool((keep[:, l] == want[l][0]).all()), l
    for pair in gs:
        for g in pair:
            g.free()
    for d in whole + [s for row in shards for s in row]:
        d.free()


def test_unpacking_fused_into_the_next_matvec():
    """Four gather objects in rotation, every matvec unpacking the previous call's gathered
    result in passing (`unpack=`): each plain buffer must hold exactly what a separate wait
    gives, i.e. the single-GPU result."""
    import torch
    from oxillama_b200.device import DeviceWeights, check_device_status
    from oxillama_b200.sharded import PeerGather
    world, rows, cols, calls = 4, 1024, 2048, 24
    w = S.gen_weight(S.Q4_K, rows, cols, seed=95)
    whole = DeviceWeights(S.Q4_K, w, rows, cols)
    shards = _shards(S.Q4_K, w, rows, cols, world)
    xs = [torch.from_numpy(S.gen_acts(1, cols, seed=95, stream=2000 + i)).cuda() for i in range(calls)]
    want = torch.empty((calls, rows), device="cuda")
    for i in range(calls):
        whole.gemm(xs[i], want[i:i + 1], 1)
    objs = [PeerGather.local_world(rows // world, world) for _ in range(4)]   # objs[slot][rank]
    got = torch.empty((calls, world, rows), device="cuda")
    for i in range(calls):
        for r in range(world):
            objs[i % 4][r].gemm(shards[r], xs[i], 1, unpack=objs[(i - 1) % 4][r] if i else None)
        if i:   # call i - 1 is unpacked now (stream order): keep it before call i + 3 overwrites it
            for r in range(world):
                got[i - 1, r].copy_(objs[(i - 1) % 4][r].buffer[0])
    for r in range(world):
        objs[(calls - 1) % 4][r].wait()
        got[calls - 1, r].copy_(objs[(calls - 1) % 4][r].buffer[0])
    torch.cuda.synchronize()
    check_device_status()
    assert bool((got == want[:, None, :]).all())
    for quad in objs:
        for g in quad:
            g.free()
    for d in shards + [whole]:
        d.free()


def test_wait_that_runs_out_is_reported_and_nothing_hangs():
    """A rank that never delivers: the other rank's bounded waits give up after a quarter of a
    second, the status word reports QK_TIMEOUT (101) once and is clear afterwards, the places
    that did not arrive read as zero, and the context stays usable."""
    import time
    import torch
    from oxillama_b200.device import DeviceWeights
    from oxillama_b200.kernels import QuantError, default_context
    from oxillama_b200.sharded import PeerGather
    ctx = default_context()
    world, rows, cols = 2, 128, 512
    w = S.gen_weight(S.Q4_K, rows, cols, seed=93)
    shards = _shards(S.Q4_K, w, rows, cols, world)
    ranks = PeerGather.local_world(rows // world, world)
    x = torch.from_numpy(S.gen_acts(1, cols, seed=93)).cuda()
    ranks[0].gemm(shards[0], x, 1)          # rank 1 never makes its call
    t0 = time.perf_counter()
    ranks[0].wait()                         # unpacking wait: rank 1's block never arrives
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    st = ctx.lib.qk_check_device_status(ctx.handle, None)
    assert st == 101, st
    assert ctx.lib.qk_check_device_status(ctx.handle, None) == 0
    got = ranks[0].buffer[0].cpu().numpy()
    assert np.all(got[rows // world:] == 0.0) and np.any(got[: rows // world] != 0.0)
    # the same for a kernel that reads its activations out of the slots
    w2 = S.gen_weight(S.Q4_K, 64, rows, seed=94)
    d2 = DeviceWeights(S.Q4_K, w2, 64, rows)
    solo = PeerGather.local_world(64, 1)[0]
    t0 = time.perf_counter()
    solo.gemm(d2, ranks[0].buffer, 1, after=ranks[0])
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    with pytest.raises(QuantError) as e:
        ctx.check(ctx.lib.qk_check_device_status(ctx.handle, None))
    assert e.value.kind == "Timeout"
    # the context is still good: an ordinary call works and reports no error
    y = torch.empty(64, device="cuda")
    d2.gemv(torch.ones(rows, device="cuda"), y)
    torch.cuda.synchronize()
    assert ctx.lib.qk_check_device_status(ctx.handle, None) == 0
    assert bool(torch.isfinite(y).all())
    solo.free()
    for g in ranks:
        g.free()
    for d in shards + [d2]:
        d.free()


def test_device_handle_entry_points_take_empty_shapes():
    """A (rows, 0) shard through the device-handle entry points: zeros, no fault."""
    import ctypes as C
    import torch
    from oxillama_b200.device import DeviceWeights, check_device_status
    from oxillama_b200.kernels import default_context
    from oxillama_b200.sharded import PeerGather
    ctx = default_context()
    dw = DeviceWeights(S.Q4_K, np.zeros(0, np.uint8), 16, 0)
    x = torch.zeros(4, device="cuda")
    y = torch.full((16,), 5.0, device="cuda")
    st = ctx.lib.qk_gemm_dev_noalloc(ctx.handle, dw.handle, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()),
                                     1, 16, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    assert bool((y == 0).all())
    pg = PeerGather(16)
    pg.gemm(dw, x, 1)
    pg.wait()
    torch.cuda.synchronize()
    check_device_status()
    assert bool((pg.buffer[0] == 0).all())
    pg.free()
    dw.free()


def test_multi_gpu_check_script():
    """With two or more GPUs visible: the multi-process check (one rank per GPU over NVLink)."""
    import os
    import subprocess
    import sys
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("one GPU visible: the in-process ranks above cover the protocol")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={min(n, 8)}",
                        "--master-addr", "127.0.0.1", "--master-port", "29541",
                        os.path.join(here, "multi_gpu_check.py")], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
