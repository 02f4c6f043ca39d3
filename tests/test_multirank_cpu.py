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


def _tp_dp_worker(rank, port, out):
    """4 gloo ranks = 2 data-parallel groups x attention-TP 2; the layer is replaced by a token-wise function with a
    cross-rank step (an all-reduce of a per-rank checksum over the expert group), so that what is checked is the glue:
    which tokens each rank feeds, and where its outputs land."""
    from hopper_megamoe_basedondeepgemm_b200 import tp_dp
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=4)
    tp_group = tp_dp.make_tp_groups(4, 2, rank)
    dp_rank, tp_rank = rank // 2, rank % 2
    m, h = 6, 8
    g = torch.Generator().manual_seed(100 + dp_rank)
    full = torch.randn((m, h), generator=g)                              # the TP group's finished hidden states
    part = torch.randn((m, h), generator=torch.Generator().manual_seed(200 + rank))
    hidden_partial = part if tp_rank == 0 else full - torch.randn((m, h), generator=torch.Generator().manual_seed(200 + rank - 1))
    seen = {}

    def layer_fn(y, hloc):
        seen['h'] = hloc.clone()
        chk = hloc.sum().reshape(1).clone()
        dist.all_reduce(chk)                                             # every rank of the expert group takes part
        y.copy_(hloc * 2.0 + 1.0)
        seen['chk'] = chk
    res = {}
    for mode in (False, True):
        y = tp_dp.moe_layer_tp_dp(hidden_partial, layer_fn, tp_group, broadcast_output=mode)
        res[mode] = y.clone()
    torch.save({'y': res[False], 'y_b': res[True], 'h': seen['h'], 'full': full, 'chk': seen['chk']}, out + f'.{rank}')
    dist.barrier()
    dist.destroy_process_group()


def test_tp_reduce_scatter_layer_all_gather_glue(tmp_path):
    out = str(tmp_path / 'tpdp')
    mp.spawn(_tp_dp_worker, args=(29543, out), nprocs=4, join=True)
    got = [torch.load(out + f'.{r}') for r in range(4)]
    total = sum(float(g['full'].sum()) for g in got[::2])
    for r in range(4):
        full, tp_rank = got[r]['full'], r % 2
        assert torch.allclose(got[r]['h'], full[tp_rank * 3:(tp_rank + 1) * 3], atol=1e-5)      # its share of the summed tokens
        assert torch.allclose(got[r]['y'], full * 2.0 + 1.0, atol=1e-5)                          # all tokens back, in order
        assert torch.allclose(got[r]['y_b'], got[r]['y'], atol=1e-6)
        assert abs(float(got[r]['chk']) - total) < 1e-3
