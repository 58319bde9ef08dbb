"""Multi-GPU parity check of the row-sharded layer (run under torchrun, one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 tests/multi_gpu_check.py

Every rank uploads its row shard, runs the sharded matvec / small matmul with the
peer-store gather (`qk_gemm_gather_dev`) and with an NCCL all-gather, and compares both
with the oracle's result for the whole matrix; then two chained sharded layers, an
expert-sharded mixture of experts summed by NCCL, and the same layer with the tokens sharded
as well (routed rows exchanged by NCCL's all-to-all).  Exits non-zero on a mismatch.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import oracle_lib as O  # noqa: E402
from oxillama_b200 import synth as S  # noqa: E402
from oxillama_b200.device import DeviceWeights, check_device_status  # noqa: E402
from oxillama_b200.sharded import PeerGather, shard_rows  # noqa: E402


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world, rank = dist.get_world_size(), dist.get_rank()
    bad = 0
    for t, rows, cols, m in ((S.Q4_K, 64 * world, 1024, 1), (S.Q4_K, 64 * world, 1024, 3), (S.Q6_K, 32 * world, 512, 1),
                             (S.Q8_0, 48 * world, 512, 9)):
        w = S.gen_weight(t, rows, cols, seed=71)
        x = S.gen_acts(m, cols, seed=71)
        st, ref = O.gemm(t, w, x, m, rows, cols)
        b, e = shard_rows(rows, world, rank)
        dw = DeviceWeights(t, w, rows, cols, b, e)
        xd = torch.from_numpy(x).cuda()
        pg = PeerGather(e - b, m_cap=m)
        for call in range(3):  # the call counting across repeated calls
            pg.gemm(dw, xd * (call + 1), m)
            pg.wait()
            torch.cuda.synchronize()
            got = pg.buffer[:m].cpu().numpy()
            err = np.abs(got - ref * (call + 1)).max() / np.abs(ref).max() / (call + 1)
            tol = 2e-5 if m <= 4 else 1e-3
            if not err <= tol:
                bad += 1
                blocks = [float(np.abs(got[:, r * (e - b):(r + 1) * (e - b)]).max()) for r in range(world)]
                print(f"rank {rank}: {S.NAMES[t]} m={m} call {call}: gather err {err}; max |y| per rank block {blocks}",
                      flush=True)
            dist.barrier()  # the next call overwrites every rank's buffer: all must have read this one
        check_device_status()
        # the NCCL route for comparison
        yl = torch.empty((m, e - b), device="cuda")
        dw.gemm(xd, yl, m)
        parts = [torch.empty_like(yl) for _ in range(world)]
        dist.all_gather(parts, yl)
        err = np.abs(torch.cat(parts, dim=1).cpu().numpy() - ref).max() / np.abs(ref).max()
        if not err <= (2e-5 if m <= 4 else 1e-3):
            bad += 1
            print(f"rank {rank}: {S.NAMES[t]} m={m}: nccl err {err}", flush=True)
        pg.free()
        dw.free()
    # two chained sharded layers: the second reads the first's gathered output and waits for it in-kernel
    for t2 in (S.Q4_K, S.Q8_0):
        n1, k1, n2 = 512, 512, 64 * world
        w1, w2 = S.gen_weight(S.Q4_K, n1, k1, seed=72), S.gen_weight(t2, n2, n1, seed=73)
        x = S.gen_acts(1, k1, seed=72)
        ref1 = O.gemm(S.Q4_K, w1, x, 1, n1, k1)[1]
        ref2 = O.gemm(t2, w2, ref1, 1, n2, n1)[1]
        b1, e1 = shard_rows(n1, world, rank)
        b2, e2 = shard_rows(n2, world, rank)
        d1, d2 = DeviceWeights(S.Q4_K, w1, n1, k1, b1, e1), DeviceWeights(t2, w2, n2, n1, b2, e2)
        g1, g2 = PeerGather(e1 - b1), PeerGather(e2 - b2)
        xd = torch.from_numpy(x).cuda()
        for call in range(3):
            g1.gemm(d1, xd, 1)
            g2.gemm(d2, g1.buffer, 1, after=g1)
            g2.wait()
            torch.cuda.synchronize()
            err = np.abs(g2.buffer[:1].cpu().numpy() - ref2).max() / np.abs(ref2).max()
            if not err <= 1e-4:
                bad += 1
                print(f"rank {rank}: chained {S.NAMES[t2]} call {call}: err {err}", flush=True)
            dist.barrier()  # nobody starts the next round while a rank still reads this one
        check_device_status()
        g1.free(), g2.free(), d1.free(), d2.free()
    # A decode chain as a model runs it: eight sharded layers, each reading the gathered output
    # of the one before it straight from the arriving slots, two gather objects alternating,
    # no host synchronisation between the layers or between repeats.  Every layer's gathered
    # result must equal, bit for bit, what one GPU computes for the whole matrix.
    n, layers, repeats = 64 * world, 8, 60
    ws = [S.gen_weight(S.Q4_K, n, n if l else 512, seed=75, stream=l, d_range=(1e-3, 2e-3)) for l in range(layers)]
    x0 = torch.from_numpy(S.gen_acts(1, 512, seed=75)).cuda()
    whole = [DeviceWeights(S.Q4_K, ws[l], n, n if l else 512) for l in range(layers)]
    want, cur = [], x0
    for l in range(layers):
        y = torch.empty((1, n), device="cuda")
        whole[l].gemm(cur, y, 1)
        want.append(y)
        cur = y
    b, e = shard_rows(n, world, rank)
    shards = [DeviceWeights(S.Q4_K, ws[l], n, n if l else 512, b, e) for l in range(layers)]
    gs = [PeerGather(e - b) for _ in range(2)]
    keep = torch.empty((repeats, layers, n), device="cuda")
    for rep in range(repeats):
        for l in range(layers):
            g, prev = gs[l & 1], gs[(l + 1) & 1]
            if l == 0:
                # the first layer of a repeat overwrites gs[0]: the last layer of the previous
                # repeat, which read it, has been waited for below by every rank
                g.gemm(shards[0], x0, 1)
            else:
                g.gemm(shards[l], prev.buffer, 1, after=prev)
            g.wait()
            keep[rep, l].copy_(g.buffer[0])
    torch.cuda.synchronize()
    check_device_status()
    for l in range(layers):
        if not bool((keep[:, l] == want[l][0]).all()):
            bad += 1
            print(f"rank {rank}: decode chain layer {l}: gathered values differ from the single-GPU result", flush=True)
    for g in gs:
        g.free()
    for d in whole + shards:
        d.free()
    # expert-sharded mixture of experts: each rank runs its experts, NCCL sums the outputs
    from oxillama_b200 import moe
    for t in (S.Q4_K, S.IQ4_XS):
        hidden, inter, n_exp, top_k, tokens = 256, 512, 8, 2, 24
        gate = [S.gen_weight(t, inter, hidden, seed=74, stream=3 * e) for e in range(n_exp)]
        up = [S.gen_weight(t, inter, hidden, seed=74, stream=3 * e + 1) for e in range(n_exp)]
        down = [S.gen_weight(t, hidden, inter, seed=74, stream=3 * e + 2) for e in range(n_exp)]
        rng = np.random.default_rng(74)
        logits = rng.standard_normal((tokens, n_exp)).astype(np.float32)
        x = rng.standard_normal((tokens, hidden)).astype(np.float32)
        deq = lambda ws, r, c: np.stack([O.dequant_matrix(t, w, r, c) for w in ws])
        ref = O.moe_ffn_f32(deq(gate, inter, hidden), deq(up, inter, hidden), deq(down, hidden, inter), logits, x, top_k)
        b, e = moe.expert_range(n_exp, world, rank)
        ex = moe.MoeExperts(t, gate[b:e], up[b:e], down[b:e], hidden, inter, n_exp, expert_begin=b)
        lg, xd = torch.from_numpy(logits).cuda(), torch.from_numpy(x).cuda()

        def local_forward(lg_, x_, k_):
            y = torch.empty((tokens, hidden), device="cuda")
            ex.forward(lg_, x_, y, k_)
            return y

        layer = moe.ExpertShardedMoe(n_exp, world, rank, local_forward)
        y = layer.forward(lg, xd, top_k)
        torch.cuda.synchronize()
        err = np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()
        if not err <= 2e-3:
            bad += 1
            print(f"rank {rank}: expert-sharded MoE {S.NAMES[t]}: err {err}", flush=True)
        check_device_status()
        # the same layer with the tokens sharded too: rank r owns a ragged share of them (the last
        # rank none when there are several), routed rows cross by NCCL's all-to-all and come back
        cuts = [round(tokens * r / max(world - 1, 1)) for r in range(world)] + [tokens] if world > 1 else [0, tokens]
        lo, hi = cuts[rank], cuts[rank + 1]

        def rows_forward(lg_, x_, k_):
            y = torch.empty((x_.shape[0], hidden), device="cuda")
            ex.forward(lg_, x_, y, k_)
            return y

        xch = moe.TokenExchangeMoe(n_exp, world, rank, rows_forward)
        y = xch.forward(lg[lo:hi].contiguous(), xd[lo:hi].contiguous(), top_k)
        torch.cuda.synchronize()
        if tuple(y.shape) != (hi - lo, hidden):
            bad += 1
            print(f"rank {rank}: token-exchange MoE {S.NAMES[t]}: shape {tuple(y.shape)}", flush=True)
        elif hi > lo:
            err = np.abs(y.cpu().numpy() - ref[lo:hi]).max() / np.abs(ref).max()
            if not err <= 2e-3:
                bad += 1
                print(f"rank {rank}: token-exchange MoE {S.NAMES[t]}: err {err}", flush=True)
        check_device_status()
        ex.free()
    tot = torch.tensor([bad], device="cuda")
    dist.all_reduce(tot)
    if rank == 0:
        print("multi_gpu_check:", "OK" if int(tot) == 0 else f"{int(tot)} mismatches", f"on {world} GPUs", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(tot) == 0 else 1)


if __name__ == "__main__":
    main()
