"""Token exchange of an expert-sharded MoE layer on the GPU, against the CPU oracle.

Every rank owns its own tokens and a range of experts; routed rows go to the experts'
ranks and the partial outputs come back (crates/oxillama-arch/src/common/moe.rs:184-258 is
the single-process layer this shards).  Here the ranks live in one process on one GPU and
the test moves the rows between them itself, in the order an all-to-all delivers them; the
run over several GPUs with NCCL's all-to-all is `tests/multi_gpu_check.py`.
"""
import numpy as np
import pytest

import oracle_lib as O
from oxillama_b200 import synth as S
from test_gpu_parity import TOL, _moe_case, rel_inf

pytestmark = pytest.mark.gpu


def test_take_rows_and_sum_rows_are_exact():
    import torch
    from oxillama_b200 import moe
    rng = np.random.default_rng(5)
    for width in (1, 7, 256, 4096):
        x = rng.standard_normal((37, width)).astype(np.float32)
        idx = rng.integers(0, 37, size=53).astype(np.int32)
        got = moe.take_rows(torch.from_numpy(x).cuda(), torch.from_numpy(idx).cuda())
        assert np.array_equal(got.cpu().numpy(), x[idx])
        table = rng.integers(-1, 37, size=(19, 3)).astype(np.int32)
        table[4] = -1  # a token nothing came back for: zeros
        want = np.zeros((19, width), dtype=np.float32)
        for t in range(19):
            for j in table[t]:
                if j >= 0:
                    want[t] = want[t] + x[j]  # f32 adds in table order
        got = moe.sum_rows(torch.from_numpy(x).cuda(), torch.from_numpy(table).cuda(), width)
        assert np.array_equal(got.cpu().numpy(), want)
    empty = moe.take_rows(torch.zeros((4, 8), device="cuda"), torch.zeros((0,), dtype=torch.int32, device="cuda"))
    assert tuple(empty.shape) == (0, 8)


def _run_ranks(layers, logits_parts, x_parts, top_k):
    """Drives the ranks' three phases in lock-step, delivering rows as an all-to-all would:
    rank r receives, in rank order, what every rank packed for it."""
    import torch
    world = len(layers)
    sent = [layer.begin(lg, x, top_k) for layer, lg, x in zip(layers, logits_parts, x_parts)]
    offs = [np.concatenate(([0], np.cumsum(st["send_counts"]))) for _, _, st in sent]
    parts = []
    for r in range(world):
        rx = torch.cat([sent[s][0][offs[s][r]:offs[s][r + 1]] for s in range(world)])
        rl = torch.cat([sent[s][1][offs[s][r]:offs[s][r + 1]] for s in range(world)])
        parts.append(layers[r].compute(rl.contiguous(), rx.contiguous(), top_k))
    outs = []
    for s in range(world):
        back = []
        for r in range(world):  # what rank r computed for rank s's rows sits behind ranks < s's rows
            begin = sum(sent[q][2]["send_counts"][r] for q in range(s))
            back.append(parts[r][begin:begin + sent[s][2]["send_counts"][r]])
        outs.append(layers[s].finish(torch.cat(back).contiguous(), sent[s][2]))
    torch.cuda.synchronize()
    return outs


@pytest.mark.parametrize("t,tokens,world,split", [
    (S.Q4_K, 40, 2, (25, 15)),      # ragged shares; grouped route on the receivers
    (S.Q4_K, 12, 2, (12, 0)),       # a rank without tokens; decode-sized receivers
    (S.IQ4_XS, 70, 4, (20, 0, 33, 17)),
    (S.Q6_K, 33, 1, (33,)),         # one rank: the exchange is the identity
])
def test_token_exchange_ranks_in_one_process(t, tokens, world, split):
    import torch
    from oxillama_b200 import moe
    from oxillama_b200.device import check_device_status
    hidden, inter, n_exp, top_k = 256, 512, 4, 2
    gate, up, down, logits, x, gf, uf, df = _moe_case(t, hidden, inter, n_exp, tokens, seed=71)
    ref = O.moe_ffn_f32(gf, uf, df, logits, x, top_k)
    experts, layers = [], []
    for r in range(world):
        b, e = moe.expert_range(n_exp, world, r)
        ex = moe.MoeExperts(t, gate[b:e], up[b:e], down[b:e], hidden, inter, n_exp, expert_begin=b)

        def local_forward(lg, xr, k, ex=ex):
            y = torch.full((xr.shape[0], hidden), float("nan"), device="cuda")
            ex.forward(lg, xr, y, k)
            return y
        experts.append(ex)
        layers.append(moe.TokenExchangeMoe(n_exp, world, r, local_forward))
    bounds = np.concatenate(([0], np.cumsum(split)))
    lgp = [torch.from_numpy(logits[bounds[r]:bounds[r + 1]].copy()).cuda() for r in range(world)]
    xp = [torch.from_numpy(x[bounds[r]:bounds[r + 1]].copy()).cuda() for r in range(world)]
    outs = _run_ranks(layers, lgp, xp, top_k)
    check_device_status()
    got = np.concatenate([o.cpu().numpy() for o in outs])
    assert got.shape == ref.shape and np.all(np.isfinite(got))
    assert rel_inf(got, ref) <= 2 * TOL  # the bar of the expert-sharded layer: three chained matmuls
    for ex in experts:
        ex.free()
