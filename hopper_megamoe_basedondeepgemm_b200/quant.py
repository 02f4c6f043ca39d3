"""Torch-side quantisation and load-time weight layout helpers (run on whatever device the tensors live on).

These mirror the casting helpers the reference's harness uses around its operator
(`sm100_b200/test_mega_moe.py:66-98,145-165`, `deep_gemm/utils/math.py`): E2M1 values with a per-32 UE8M0 scale
(MXFP4) or a per-16 UE4M3 scale (NVFP4). They are load-time / test-input utilities; the hot path is the CUDA kernel.
"""
from typing import Tuple

import torch

SF_VEC = {'mxfp4': 32, 'nvfp4': 16, 'fp8': 32}
_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_TIE_UP = (False, True, False, True, False, True, False)


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """2^ceil(log2|x|) with the exponent clamped to [1, 254] (`deep_gemm/utils/math.py:13-16`)."""
    bits = x.abs().float().contiguous().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (exp.clamp(1, 254) << 23).view(torch.float32)


def quantize_to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 codes (uint8), round to nearest even, saturating at +-6."""
    ax = x.abs()
    code = torch.zeros_like(x, dtype=torch.uint8)
    for b, up in zip(_BOUNDS, _TIE_UP):
        code += ((ax >= b) if up else (ax > b)).to(torch.uint8)
    return code | (torch.signbit(x).to(torch.uint8) << 3)


def cast_rows_to_fp4(t: torch.Tensor, fmt: str, global_scale: float = 1.0
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[M, K] -> (packed int8 [M, K/2], scales fp32 [M, K/vec], scales int32 [M, K/(4 vec)], 4 scale bytes per word).

    The layout of `cast_to_fp4_rows` (`sm100_b200/test_mega_moe.py:78-93`); `global_scale` divides the tensor first
    (NVFP4 per-tensor scale).
    """
    vec = SF_VEC[fmt]
    m, k = t.shape
    g = (t.float() / global_scale).view(m, k // vec, vec)
    amax = g.abs().amax(dim=-1).clamp_min(1e-30)
    if fmt == 'nvfp4':
        sf = (amax / 6.0).to(torch.float8_e4m3fn).float()
        sf_b = sf.to(torch.float8_e4m3fn).view(torch.uint8)
        scaled = torch.nan_to_num(g / sf.unsqueeze(-1), nan=0.0, posinf=6.0, neginf=-6.0)
    else:
        sf = ceil_to_ue8m0(amax / 6.0)
        sf_b = (sf.view(torch.int32) >> 23).to(torch.uint8)
        scaled = g / sf.unsqueeze(-1)
    codes = quantize_to_e2m1(scaled).view(m, k)
    packed = ((codes[:, 0::2] & 0xF) | ((codes[:, 1::2] & 0xF) << 4)).contiguous().view(torch.int8)
    return packed, sf, sf_b.contiguous().view(torch.int32)


def cast_rows_to_fp8(t: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[M, K] -> (E4M3 [M, K], scales fp32 [M, K/32], scales int32 [M, K/128], 4 UE8M0 bytes per word).

    `per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32)` of `deep_gemm/utils/math.py:26-38`: block maxima clamped at
    1e-4, scale 2^ceil(log2(amax / 448)).
    """
    m, k = t.shape
    g = t.float().view(m, k // 32, 32)
    amax = g.abs().amax(dim=-1).clamp_min(1e-4)
    sf = ceil_to_ue8m0(amax / 448.0)
    sf_b = (sf.view(torch.int32) >> 23).to(torch.uint8)
    q = (g * (1.0 / sf.unsqueeze(-1))).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(m, k)
    return q, sf, sf_b.contiguous().view(torch.int32)


def cast_grouped_weights_to_fp4(w: torch.Tensor, fmt: str, global_scale: float = 1.0
                                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [E, N, K] -> (packed int8 [E, N, K/2], scales int32 [E, N, K/(4 vec)] stored MN-major).

    The operator's weight input convention (`sm100_b200/test_mega_moe.py:158-165`): the scale tensor has strides
    (K/(4 vec) * N, 1, N).
    """
    wfmt = 'mxfp4' if fmt == 'fp8' else fmt
    vec = SF_VEC[wfmt]
    e, n, k = w.shape
    q = torch.empty((e, n, k // 2), dtype=torch.int8, device=w.device)
    sf_mn = torch.empty((e, k // (4 * vec), n), dtype=torch.int32, device=w.device).permute(0, 2, 1)
    for i in range(e):
        q[i], _, s = cast_rows_to_fp4(w[i], wfmt, global_scale)
        sf_mn[i].copy_(s)
    return q, sf_mn


def interleave_gate_up(t: torch.Tensor, gran: int = 8) -> torch.Tensor:
    """[E, 2I, ...] rows [gate | up] -> groups of `gran` gate rows followed by the matching `gran` up rows
    (`sm100_b200/mega___init__.py:81-90`)."""
    e, n = t.shape[:2]
    rest = t.shape[2:]
    half = n // 2
    gate = t[:, :half].reshape(e, half // gran, gran, *rest)
    up = t[:, half:].reshape(e, half // gran, gran, *rest)
    return torch.stack([gate, up], dim=2).reshape(e, n, *rest).contiguous()


def pretile_weights(w_packed: torch.Tensor, sf_words: torch.Tensor, vec: int) -> torch.Tensor:
    """Lay one grouped weight tensor out as the stream the kernel copies into shared memory verbatim.

    Input: packed E2M1 [E, N, K/2] (K-major) and scale words int32 [E, N, K/(4 vec)] (any strides).
    Output uint8 [E, N/128, K/256, unit_bytes]: for each (expert, 128-row tile, 256-element K unit) the 128 x 128 B
    weight block in the 128 B-swizzled shared-memory image (16 B chunk c of row r at chunk position c ^ (r % 8)),
    followed by the unit's scale planes, one 512 B plane per scale word: word index (r % 32) * 4 + r / 32
    (the 32-lane x 4-column order of the tensor-memory scale copy; the reference applies the same 4 x 32 transpose
    to its scale tensors, `sm100_b200/mega___init__.py:93-99`).
    """
    e, n, kh = w_packed.shape
    k = kh * 2
    assert n % 128 == 0 and k % 256 == 0, 'weight rows must be a multiple of 128 and K of 256'
    nt, ku, planes = n // 128, k // 256, 256 // (4 * vec)
    dev = w_packed.device
    w = w_packed.contiguous().view(torch.uint8).reshape(e, nt, 128, ku, 8, 16).permute(0, 1, 3, 2, 4, 5)
    r = torch.arange(128, device=dev)
    src_chunk = torch.arange(8, device=dev)[None, :] ^ (r[:, None] % 8)
    w = w[:, :, :, r[:, None], src_chunk, :].reshape(e, nt, ku, 128 * 128)
    sf = sf_words.contiguous().view(torch.uint8).reshape(e, nt, 4, 32, ku, planes, 4)     # [e, tile, a, b, unit, plane, byte]
    sf = sf.permute(0, 1, 4, 5, 3, 2, 6).reshape(e, nt, ku, planes * 512)
    return torch.cat([w, sf], dim=-1).contiguous()
