"""Shared helpers of the parity tests: seeded workloads in the oracle's and in the operator's formats."""
import torch

from oracle import megamoe_oracle as O


def sf_to_bytes(sf: torch.Tensor, fmt: str) -> torch.Tensor:
    return O.ue4m3_byte(sf) if fmt == 'nvfp4' else O.ue8m0_byte(sf)


def to_operator_weights(w: O.RankWeights, fmt: str, device):
    """Oracle weights -> the operator's input convention (packed int8, MN-major int32 scale words)."""
    wfmt = 'mxfp4' if fmt == 'fp8' else fmt

    def one(q, sf):
        e, n, kh = q.shape
        words = sf_to_bytes(sf, wfmt).contiguous().view(torch.int32)              # [E, N, K/(4 vec)]
        sf_mn = torch.empty((e, words.shape[-1], n), dtype=torch.int32).permute(0, 2, 1)
        sf_mn.copy_(words)
        return q.view(torch.int8).to(device), sf_mn.to(device)
    return one(w.w1_q, w.w1_sf), one(w.w2_q, w.w2_sf)


def make_rank_inputs(num_tokens, hidden, fmt, seed, topk_idx, topk_weights, x_global_scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((num_tokens, hidden), generator=g).to(torch.bfloat16)
    q, sf, sfb = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul', global_scale=x_global_scale)
    return x, O.RankInput(q, sf, topk_idx, topk_weights), sfb


def random_routing(num_tokens, num_experts, topk, seed, masked_ratio=0.0):
    g = torch.Generator().manual_seed(seed)
    scores = torch.randn((num_tokens, num_experts), generator=g)
    w, idx = torch.topk(scores, topk, dim=-1, largest=True, sorted=False)
    w = torch.softmax(w, dim=-1)
    if masked_ratio > 0:
        m = torch.rand(idx.shape, generator=g) < masked_ratio
        idx = idx.masked_fill(m, -1)
        w = w.masked_fill(m, 0.0)
    return idx, w.float()


def write_inputs(buf, inp: O.RankInput, sfb: torch.Tensor):
    t = inp.x_q.shape[0]
    if t == 0:
        return
    buf.x[:t].copy_(inp.x_q.view(buf.x.dtype))
    buf.x_sf[:t].copy_(sfb.contiguous().view(torch.int32))
    buf.topk_idx[:t].copy_(inp.topk_idx)
    buf.topk_weights[:t].copy_(inp.topk_weights)


def last_cuda_error() -> str:
    """Text of the latest CUDA runtime failure the library recorded (empty if none)."""
    import ctypes
    from hopper_megamoe_basedondeepgemm_b200 import _lib
    lib = _lib.load()
    lib.mm_last_cuda_error.restype = ctypes.c_char_p
    msg = lib.mm_last_cuda_error()
    return msg.decode() if msg else ''
