"""Host-side multi-rank logic on CPU: two gloo ranks compute their experts' share of the layer like the reference's
test does (all-gather inputs, all-reduce partial outputs, `sm100_b200/test_mega_moe.py:442-486`) and must reproduce the
single-process oracle."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import megamoe_oracle as O
from tests import util_moe as U

FMT, E_LOCAL, HIDDEN, INTER, TOPK, WORLD = 'mxfp4', 4, 512, 256, 2, 2
TOKENS = [3, 2]


def _inputs():
    ins, ws = [], []
    for r in range(WORLD):
        idx, tw = U.random_routing(TOKENS[r], E_LOCAL * WORLD, TOPK, 10 + r, masked_ratio=0.1)
        _, inp, _ = U.make_rank_inputs(TOKENS[r], HIDDEN, FMT, 20 + r, idx, tw)
        ins.append(inp)
        ws.append(O.make_expert_weights(E_LOCAL, HIDDEN, INTER, FMT, seed=30 + r, std=0.05)[0])
    return ins, ws


def _worker(rank, port, out):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=WORLD)
    ins, ws = _inputs()
    mine = ins[rank]
    x_dq = O.dequant_fp4_rows(mine.x_q, mine.x_sf, 32)
    # uneven all-gather of tokens and routing (pad to the largest rank)
    tmax = max(TOKENS)
    def gather(t, fill):
        pad = torch.full((tmax,) + tuple(t.shape[1:]), fill, dtype=t.dtype)
        pad[:t.shape[0]] = t
        outl = [torch.empty_like(pad) for _ in range(WORLD)]
        dist.all_gather(outl, pad)
        return torch.cat([o[:TOKENS[r]] for r, o in enumerate(outl)])
    X, IDX, W = gather(x_dq, 0.0), gather(mine.topk_idx, -1), gather(mine.topk_weights, 0.0)
    y = torch.zeros((X.shape[0], HIDDEN))
    counts = torch.zeros(E_LOCAL, dtype=torch.int32)
    for el in range(E_LOCAL):
        e = rank * E_LOCAL + el
        t_ids, s_ids = torch.nonzero(IDX == e, as_tuple=True)
        counts[el] = t_ids.numel()
        if t_ids.numel() == 0:
            continue
        w1 = O.dequant_fp4_rows(ws[rank].w1_q[el], ws[rank].w1_sf[el], 32)
        w2 = O.dequant_fp4_rows(ws[rank].w2_q[el], ws[rank].w2_sf[el], 32)
        act = O.swiglu_weighted(X[t_ids] @ w1.t(), INTER, 10.0, W[t_ids, s_ids])
        q, sf, _ = O.quant_fp4_rows(act, FMT, rounding='rne', sf_rule='div')
        y.index_add_(0, t_ids, O.dequant_fp4_rows(q, sf, 32) @ w2.t())
    dist.all_reduce(y)
    start = sum(TOKENS[:rank])
    torch.save({'y': y[start:start + TOKENS[rank]], 'counts': counts}, out + f'.{rank}')
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_process_oracle(tmp_path):
    out = str(tmp_path / 'res')
    mp.spawn(_worker, args=(29541, out), nprocs=WORLD, join=True)
    ins, ws = _inputs()
    ref = O.moe_layer_reference(ins, ws, FMT, E_LOCAL * WORLD, clamp=10.0, faithful=False, rounding='rne')
    for r in range(WORLD):
        got = torch.load(out + f'.{r}')
        assert torch.equal(got['counts'], ref.counts[r])
        assert torch.equal(got['y'].to(torch.bfloat16), ref.y[r])
