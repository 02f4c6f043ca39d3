"""Caller-side glue for data-parallel attention with tensor-parallel attention groups around the layer.

The reference's serving entry wraps its MegaMoE call the same way (`deep_gemm/mega/__init__.py:396-443,492-507`,
benchmarked by `tests/bench_customer_bs2_tp4_dp2.py`: "TP ReduceScatter -> fused MegaMoE -> token AllGather"): the
ranks of one attention-TP group hold partial sums of the same token stream; a reduce-scatter leaves every rank with
the finished hidden states of its 1/tp share of the tokens, the expert-parallel layer runs on those shares over the
whole expert group, and an all-gather inside the TP group restores the full token stream for the next attention block.
Rank layout: data-parallel outer, attention-TP inner (`ep_rank % tp_size == tp_rank`), as the reference asserts.
"""
from typing import Callable, Optional

import torch
import torch.distributed as dist


def make_tp_groups(world_size: int, tp_size: int, rank: int):
    """One process group per run of `tp_size` consecutive ranks (every rank must call this); returns this rank's group
    (`tests/bench_customer_bs2_tp4_dp2.py:23-31`)."""
    mine = None
    for first in range(0, world_size, tp_size):
        ranks = list(range(first, first + tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            mine = g
    return mine


def _reduce_scatter_tokens(out: torch.Tensor, partial: torch.Tensor, group) -> None:
    """out[m/tp, h] = this rank's token share of the sum of `partial` [m, h] over the group."""
    if dist.get_backend(group) == 'nccl':
        dist.reduce_scatter_tensor(out, partial, group=group)
        return
    full = partial.clone()                                    # (gloo has no reduce-scatter: all-reduce, keep the share)
    dist.all_reduce(full, group=group)
    share, r = out.size(0), dist.get_rank(group)
    out.copy_(full[r * share:(r + 1) * share])


def moe_layer_tp_dp(hidden_partial: torch.Tensor, layer_fn: Callable[[torch.Tensor, torch.Tensor], None],
                    attn_tp_group, y_full: Optional[torch.Tensor] = None, broadcast_output: bool = False) -> torch.Tensor:
    """TP reduce-scatter -> `layer_fn(y_local, hidden_local)` -> token all-gather.

    hidden_partial: bf16 [m, h], this rank's partial sum of the TP group's m tokens (m divisible by the TP size).
    layer_fn: runs the expert-parallel layer on the local share, e.g.
        `lambda y, h: mega_moe_from_hidden(y, h, router_w, l1, l2, sym_buffer, workspace, ...)`;
      every rank of the expert group calls it collectively, as the layer requires.
    Returns y_full [m, h]: the layer's output for all m tokens, identical on every rank of the TP group.
    `broadcast_output` reproduces the reference's gather-to-root + broadcast mode (same result, other traffic pattern).
    """
    tp = dist.get_world_size(attn_tp_group)
    m, h = hidden_partial.shape
    if m % tp != 0:
        raise RuntimeError('the token count must be divisible by the attention-TP size')
    local_m = m // tp
    hidden_local = torch.empty((local_m, h), dtype=hidden_partial.dtype, device=hidden_partial.device)
    _reduce_scatter_tokens(hidden_local, hidden_partial.contiguous(), attn_tp_group)
    y_local = torch.empty_like(hidden_local)
    layer_fn(y_local, hidden_local)
    if y_full is None:
        y_full = torch.empty((m, h), dtype=y_local.dtype, device=y_local.device)
    if broadcast_output:
        r = dist.get_rank(attn_tp_group)
        root = dist.get_global_rank(attn_tp_group, 0)
        y_full.zero_()
        y_full[r * local_m:(r + 1) * local_m].copy_(y_local)
        dist.reduce(y_full, dst=root, group=attn_tp_group)
        dist.broadcast(y_full, src=root, group=attn_tp_group)
    else:
        dist.all_gather_into_tensor(y_full, y_local, group=attn_tp_group)
    return y_full
