"""Seeded synthetic workloads with the shapes and value distributions of the reference's harness
(`sm100_b200/test_mega_moe.py:100-171`): bf16 tokens ~ N(0, 1), expert weights ~ N(0, std) quantised to E2M1 with
block scales, forced-balanced routing. Stand-ins for the reference's benchmark inputs; no external data is involved.
"""
from typing import Tuple

import torch

from . import quant
from .mega import transform_weights_for_mega_moe


def balanced_routing(num_tokens: int, rank: int, num_ranks: int, num_experts: int, topk: int, token_offset: int = 0,
                     device='cpu') -> Tuple[torch.Tensor, torch.Tensor]:
    """Forced-balanced routing (`sm100_b200/test_mega_moe.py:113-123`).

    One rank: expert = (g * topk + s) % E. Several ranks: g = t + rank * 1000003 and slot s goes to rank s % R,
    expert = (s % R) * E_local + (g + 7 s + 11 (s // R)) % E_local, weight 1 / topk; with 8 ranks and top-8 this is
    the reference's formula. `token_offset` shifts g (the benchmark rotates it so that successive steps touch
    different experts).
    """
    s = torch.arange(topk, dtype=torch.int64, device=device)
    t = torch.arange(num_tokens, dtype=torch.int64, device=device) + token_offset
    if num_ranks == 1:
        idx = (t[:, None] * topk + s[None, :]) % num_experts
    else:
        e_local = num_experts // num_ranks
        g = t + rank * 1000003
        r = s % num_ranks
        idx = r[None, :] * e_local + (g[:, None] + 7 * s[None, :] + (s // num_ranks)[None, :] * 11) % e_local
    w = torch.full((num_tokens, topk), 1.0 / topk, dtype=torch.float32, device=device)
    return idx, w


def make_layer_weights(e_local: int, hidden: int, inter: int, fmt: str, seed: int, std: float = 0.02, device='cuda',
                       keep_untransformed: bool = False):
    """Random expert weights -> ((l1 stream, shape), (l2 stream, shape), (l1 global scale, l2 global scale)); with
    `keep_untransformed` also the operator-format inputs of the transform [(w1, w1_sf), (w2, w2_sf)] (for checkers)."""
    g = torch.Generator(device=device).manual_seed(seed)
    out, scales = [], []
    for n, k in ((2 * inter, hidden), (hidden, inter)):
        w = (torch.randn((e_local, n, k), generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)
        gs = float(w.float().abs().max() / (6.0 * 448.0)) if fmt == 'nvfp4' else 1.0
        out.append(quant.cast_grouped_weights_to_fp4(w, fmt, gs))
        scales.append(gs)
        del w
    l1, l2 = transform_weights_for_mega_moe(out[0], out[1])
    if keep_untransformed:
        return l1, l2, tuple(scales), out
    return l1, l2, tuple(scales)


def make_tokens(num_tokens: int, hidden: int, fmt: str, seed: int, device='cuda', global_scale: float = 1.0):
    """bf16 tokens ~ N(0, 1) and their quantised form (packed E2M1 as int8, or E4M3 for 'fp8'; scale words int32)."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((num_tokens, hidden), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    packed, _, words = quant.cast_rows_to_fp8(x) if fmt == 'fp8' else quant.cast_rows_to_fp4(x, fmt, global_scale)
    return x, packed, words


def active_experts_per_rank(topk_idx_all_ranks, num_experts: int, num_ranks: int):
    """Distinct experts with at least one routed row, per destination rank (drives the algorithmic weight bytes)."""
    e_local = num_experts // num_ranks
    idx = torch.cat([i.flatten() for i in topk_idx_all_ranks])
    idx = idx[idx >= 0]
    return [int(torch.unique(idx[(idx // e_local) == r]).numel()) for r in range(num_ranks)]


def weight_bytes_per_expert(hidden: int, inter: int, fmt: str) -> int:
    """W1 + W1 scales + W2 + W2 scales of one expert: the bytes one launch must stream per active expert."""
    vec = quant.SF_VEC['mxfp4' if fmt == 'fp8' else fmt]
    return 2 * inter * hidden // 2 + 2 * inter * hidden // vec + hidden * inter // 2 + hidden * inter // vec
