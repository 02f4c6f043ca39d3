"""Multi-rank parity worker (launched by torchrun, one process per GPU, NCCL + symmetric memory).

Checks, per rank: per-expert receive counts exact, canonical slot order (through the intermediate rows), y within the
parity tolerance of the CPU oracle that simulates all ranks in one process. Prints `MP_OK` on rank 0 when every rank passed.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import hopper_megamoe_basedondeepgemm_b200 as mm          # noqa: E402
from oracle import megamoe_oracle as O                     # noqa: E402
from tests import util_moe as U                            # noqa: E402


def run_from_hidden(rank, world, group, fmt, skewed=False):
    """The whole layer from bf16 hidden states (router + top-8 + quantisation fused at the head of the kernel).
    `skewed`: sigmoid scores + Zipf(1.2) expert bias, renormalised top-8, 16 tokens per rank: the hot experts receive
    more than 16 rows (32-row token tiles), most experts few or none."""
    e_local, hidden, inter, topk = 8, 1024, 512, 8
    num_experts = e_local * world
    tokens = [16 - r for r in range(world)] if skewed else [5 + 2 * r for r in range(world)]
    ok = True
    buf = mm.get_symm_buffer_for_mega_moe(group, num_experts, 16, topk, hidden, inter, act_format=fmt)
    gb = torch.Generator().manual_seed(11)
    bias = (1.0 / torch.arange(1, num_experts + 1, dtype=torch.float32) ** 1.2)[torch.randperm(num_experts, generator=gb)] if skewed else None
    mode = 'sigmoid_bias' if skewed else 'softmax'
    weights = [O.make_expert_weights(e_local, hidden, inter, fmt, seed=70 + r, std=0.05)[0] for r in range(world)]
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(weights[rank], fmt, 'cuda'))
    ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
    g = torch.Generator().manual_seed(7)
    wr = (torch.randn((num_experts, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    for it in range(2):
        xs, inputs = [], []
        for r in range(world):
            gx = torch.Generator().manual_seed(1000 * it + r)
            x = torch.randn((tokens[r], hidden), generator=gx).to(torch.bfloat16)
            idx, tw = O.route_from_logits(O.router_logits_device_order(x, wr), x, topk, mode, bias)
            q, sf, _ = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul')
            xs.append(x); inputs.append(O.RankInput(q, sf, idx, tw))
        ref = O.moe_layer_reference(inputs, weights, fmt, num_experts, clamp=10.0)
        y = torch.empty((tokens[rank], hidden), dtype=torch.bfloat16, device='cuda')
        stats = torch.zeros(e_local, dtype=torch.int32, device='cuda')
        dist.barrier()
        mm.mega_moe_from_hidden(y, xs[rank].cuda(), wr.cuda(), l1, l2, buf, ws, cumulative_local_expert_recv_stats=stats,
                                activation_clamp=10.0, score_mode=1 if skewed else 0,
                                expert_bias=bias.cuda() if skewed else None, timeout_ms=2000.0)
        st, words = buf.device_status()
        if st != 0:
            print(f'rank {rank}: device status {st} {[hex(v) for v in words[:4]]}', flush=True)
            return False
        if not torch.equal(stats.cpu(), ref.counts[rank]):
            print(f'rank {rank} it {it}: counts {stats.cpu().tolist()} != {ref.counts[rank].tolist()}', flush=True)
            ok = False
        if skewed and rank == 0 and it == 0 and max(int(c.max()) for c in ref.counts) <= 16:
            print('the skewed case has no expert with more than 16 rows', flush=True)
            ok = False
        if not torch.equal(buf.topk_idx[:tokens[rank]].cpu(), inputs[rank].topk_idx):
            print(f'rank {rank} it {it}: top-8 differs from the oracle', flush=True)
            ok = False
        err, cos = O.rel_rmse(y.cpu(), ref.y[rank]), O.cosine(y.cpu(), ref.y[rank])
        if not (err <= 3e-3 and cos >= 0.9999):
            print(f'rank {rank} it {it}: rel_rmse {err:.4e} cos {cos:.6f}', flush=True)
            ok = False
        torch.cuda.synchronize()
        dist.barrier()
    return ok


def main():
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', rank)))
    dist.init_process_group('nccl', device_id=torch.device('cuda', torch.cuda.current_device()))
    group = dist.group.WORLD
    fmt = os.environ.get('MP_FORMAT', 'mxfp4')
    engine = os.environ.get('MP_ENGINE', 'umma')
    if os.environ.get('MP_MODE', 'routed') in ('from_hidden', 'from_hidden_skewed'):
        skewed = os.environ['MP_MODE'] == 'from_hidden_skewed'
        flag = torch.tensor([1 if run_from_hidden(rank, world, group, fmt, skewed) else 0], device='cuda')
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print('MP_OK' if int(flag) == 1 else 'MP_FAIL', flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    e_local, hidden, inter, topk = 8, 1024, 512, 4
    num_experts = e_local * world
    tokens = [(5 + 3 * r) % 7 for r in range(world)]          # ragged, some ranks may have 0 tokens
    tokens[world - 1] = 0 if world > 2 else tokens[world - 1]
    if os.environ.get('MP_TOKENS'):                            # many rows per destination: several SMs share a dispatch
        tokens = [int(os.environ['MP_TOKENS']) - 3 * r for r in range(world)]
    ok = True
    buf = mm.get_symm_buffer_for_mega_moe(group, num_experts, max(16, max(tokens)), topk, hidden, inter, act_format=fmt,
                                          window=os.environ.get('MP_WINDOW', 'symm_mem'))
    weights = [O.make_expert_weights(e_local, hidden, inter, fmt, seed=50 + r, std=0.05)[0] for r in range(world)]
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(weights[rank], fmt, 'cuda'))
    for it in range(3):                                          # consecutive launches exercise both parities
        inputs, sfbs = [], []
        for r in range(world):
            idx, tw = U.random_routing(tokens[r], num_experts, topk, 100 * it + r, masked_ratio=0.15)
            _, inp, sfb = U.make_rank_inputs(tokens[r], hidden, fmt, 200 * it + r, idx, tw)
            inputs.append(inp); sfbs.append(sfb)
        ref = O.moe_layer_reference(inputs, weights, fmt, num_experts, clamp=10.0, keep_mid=True)
        U.write_inputs(buf, inputs[rank], sfbs[rank])
        y = torch.empty((tokens[rank], hidden), dtype=torch.bfloat16, device='cuda')
        stats = torch.zeros(e_local, dtype=torch.int32, device='cuda')
        dist.barrier()
        op = mm.fp8_fp4_mega_moe if fmt == 'fp8' else mm.fp4_fp4_mega_moe
        op(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0, engine=engine, timeout_ms=2000.0)
        st, words = buf.device_status()
        if st != 0:
            print(f'rank {rank}: device status {st} {[hex(v) for v in words[:4]]}', flush=True)
            ok = False
            break
        if not torch.equal(stats.cpu(), ref.counts[rank]):
            print(f'rank {rank}: counts {stats.cpu().tolist()} != {ref.counts[rank].tolist()}', flush=True)
            ok = False
        if tokens[rank]:
            err, cos = O.rel_rmse(y.cpu(), ref.y[rank]), O.cosine(y.cpu(), ref.y[rank])
            if not (err <= 3e-3 and cos >= 0.9999):
                print(f'rank {rank} it {it}: rel_rmse {err:.4e} cos {cos:.6f}', flush=True)
                ok = False
        # slot map: the records kept in the receive pool, grouped per expert in row order, equal the canonical
        # (source rank, token, slot) order exactly
        recs = buf.received_records()
        got_map = [[] for _ in range(e_local)]
        if any(r is None or any(v is None for v in r) for r in recs):
            print(f'rank {rank} it {it}: incomplete records in the receive pool', flush=True)
            ok = False
        else:
            for src, rows in enumerate(recs):
                for (e, t, s, _) in rows:
                    got_map[e].append((src, t, s))
            if got_map != [list(v) for v in ref.slot_map[rank]]:
                print(f'rank {rank} it {it}: slot map differs from the canonical order', flush=True)
                ok = False
        # and the intermediate rows sit in that order
        vec = O.SF_VEC[fmt]
        mid, mid_sf = buf.l2_acts_payload().cpu(), buf.l2_acts_sf_payload().cpu()
        base, step = 0, buf.tile_image_rows() or 16        # rows of an expert start on a tile boundary (16 or 32 rows)
        for e, cnt in enumerate(ref.counts[rank].tolist()):
            if cnt == 0:
                continue
            deq = O.dequant_fp8_rows if fmt == 'fp8' else (lambda q, sf: O.dequant_fp4_rows(q, sf, vec))
            got = deq(mid[base:base + cnt], O.sf_bytes_to_float(mid_sf[base:base + cnt, :inter // vec], fmt))
            want = deq(ref.mid_q[rank][e], O.sf_bytes_to_float(ref.mid_sf[rank][e], fmt))
            if any(O.rel_rmse(got[n], want[n]) > 0.05 for n in range(cnt)):
                print(f'rank {rank} it {it}: expert {e} intermediate rows differ ({O.rel_rmse(got, want):.3f})', flush=True)
                ok = False
            base += (cnt + step - 1) // step * step
        torch.cuda.synchronize()
        dist.barrier()
    flag = torch.tensor([1 if ok else 0], device='cuda')
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print('MP_OK' if int(flag) == 1 else 'MP_FAIL', flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
