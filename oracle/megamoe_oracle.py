"""CPU oracle for the expert-parallel MegaMoE layer (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it. It restates, in
plain torch on CPU tensors, the pure-torch quantised MoE that the reference
uses to validate its fused kernels, plus the router / quantisation rules of the
reference's frontend. Every function cites the reference lines it follows
(paths are relative to the reference project's root).

Pinning: `tests/golden/make_golden.py` imports the reference's own helper
module (`deep_gemm/utils/math.py`) and its test formulas, runs them on seeded
inputs and stores the results under `tests/golden/`; `tests/test_oracle.py`
checks this restatement against those vectors.

Two deliberate, documented deviations are selectable by argument:
  * `rounding='rne'` (default) encodes E2M1 round-to-nearest-even, as the
    hardware `cvt.rn.satfinite.e2m1x2.f32` does; `rounding='ref'` reproduces
    the reference helper's "ties toward the smaller magnitude" rule
    (`deep_gemm/utils/math.py:73-82`).
  * `faithful=True` (default) rounds every routed expert output to bf16 and sums
    the routes of a token in ascending slot order in fp32 (what the fused kernel
    does, `sm100_b200/sm100_fp4_fp4_mega_moe.cuh:1887-1916`); `faithful=False`
    sums in fp32 without the per-route rounding like the reference's test
    (`sm100_b200/test_mega_moe.py:484-486`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

FP4_VALUES = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)
SF_VEC = {'mxfp4': 32, 'nvfp4': 16, 'fp8': 32}


# ----------------------------------------------------------------------------- scale factors
def ceil_pow2(x: torch.Tensor) -> torch.Tensor:
    """2^ceil(log2(|x|)) from the float bits, exponent clamped to [1, 254].

    Follows `deep_gemm/utils/math.py:13-16` (`ceil_to_ue8m0`).
    """
    bits = x.abs().float().contiguous().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (exp.clamp(1, 254) << 23).view(torch.float32)


def ue8m0_byte(sf: torch.Tensor) -> torch.Tensor:
    """Power-of-two fp32 scale -> its exponent byte (`sm100_b200/test_mega_moe.py:77`)."""
    return (sf.contiguous().view(torch.int32) >> 23).to(torch.uint8)


def ue4m3_round(x: torch.Tensor, floor_to_min_subnormal: bool = False) -> torch.Tensor:
    """fp32 -> E4M3 (round to nearest even) -> fp32, `sm100_b200/test_mega_moe.py:70-71`.

    `floor_to_min_subnormal` replaces an encoded zero by the smallest subnormal,
    as the frontend does (`sm100_b200/fe_sm100/fable_frontend_sm100.cu:145-147`).
    """
    q = x.float().to(torch.float8_e4m3fn)
    if floor_to_min_subnormal:
        b = q.view(torch.uint8).clone()
        b[b == 0] = 1
        q = b.view(torch.float8_e4m3fn)
    return q.float()


def ue4m3_byte(sf: torch.Tensor) -> torch.Tensor:
    return sf.float().to(torch.float8_e4m3fn).view(torch.uint8)


# ----------------------------------------------------------------------------- E2M1
_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
# On a tie the even code wins: codes (0,1)->0, (1,2)->2, (2,3)->2, (3,4)->4, (4,5)->4, (5,6)->6, (6,7)->6
_TIE_UP = (False, True, False, True, False, True, False)


def e2m1_encode(x: torch.Tensor, rounding: str = 'rne') -> torch.Tensor:
    """fp32 -> 4-bit E2M1 code (uint8, sign in bit 3), saturating at 6.

    `rounding='ref'`: `deep_gemm/utils/math.py:73-82` (`> boundary`; the sign is
    dropped for a zero magnitude). `rounding='rne'`: round to nearest even, sign
    kept (what the `cvt.rn.satfinite.e2m1x2.f32` instruction produces,
    `sm100_b200/fe_sm100/fable_frontend_sm100.cu:166-168`).
    """
    ax = x.abs()
    code = torch.zeros_like(x, dtype=torch.uint8)
    for b, up in zip(_BOUNDS, _TIE_UP):
        if rounding == 'rne' and up:
            code += (ax >= b).to(torch.uint8)
        else:
            code += (ax > b).to(torch.uint8)
    if rounding == 'ref':
        sign = (x < 0) & (code != 0)
    else:
        sign = torch.signbit(x)
    return code | (sign.to(torch.uint8) << 3)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    return FP4_VALUES[code.long()]


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[.., K] codes -> [.., K/2] bytes, even element in the low nibble (`test_mega_moe.py:91`)."""
    return ((codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4)).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    u = packed.view(torch.uint8)
    return torch.stack([u & 0xF, u >> 4], dim=-1).reshape(*u.shape[:-1], u.shape[-1] * 2)


# ----------------------------------------------------------------------------- row quantisers
def fp4_scale_for(amax: torch.Tensor, fmt: str, sf_rule: str = 'div') -> torch.Tensor:
    """Per-group scale from the group amax.

    MXFP4: 2^ceil(log2(amax / 6)); NVFP4: e4m3(amax / 6) (`test_mega_moe.py:68-72`).
    `sf_rule='div'` divides by 6 (test helper, L1 epilogue); `'mul'` multiplies by the
    fp32 constant 1/6 and never yields an NVFP4 zero scale (the frontend's
    arithmetic, `fable_frontend_sm100.cu:142-152`).
    """
    v = amax / 6.0 if sf_rule == 'div' else amax * torch.tensor(1.0 / 6.0, dtype=torch.float32)
    if fmt == 'nvfp4':
        return ue4m3_round(v, floor_to_min_subnormal=(sf_rule == 'mul'))
    return ceil_pow2(v)


def quant_fp4_rows(t: torch.Tensor, fmt: str, rounding: str = 'rne', sf_rule: str = 'div',
                   global_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[M, K] -> (packed uint8 [M, K/2], scale fp32 [M, K/vec], scale bytes uint8 [M, K/vec]).

    Follows `cast_to_fp4_rows` (`sm100_b200/test_mega_moe.py:78-93`): per-`vec`
    amax clamped at 1e-30, scale by `fp4_scale_for`, values `x / sf` encoded as
    E2M1. With `sf_rule='mul'` the values are multiplied by `1 / sf` instead
    (frontend, `fable_frontend_sm100.cu:155`). `global_scale` (NVFP4 extension,
    not in the reference's B200 kernels) divides the tensor first.
    """
    vec = SF_VEC[fmt]
    m, k = t.shape
    g = (t.float() / global_scale).view(m, k // vec, vec)
    amax = g.abs().amax(dim=-1).clamp_min(1e-30)
    sf = fp4_scale_for(amax, fmt, sf_rule)
    if sf_rule == 'mul':
        scaled = g * (1.0 / sf).unsqueeze(-1)
    else:
        scaled = g / sf.unsqueeze(-1)
    if fmt == 'nvfp4':
        scaled = torch.nan_to_num(scaled, nan=0.0, posinf=6.0, neginf=-6.0)   # sf == 0 only when the group is ~0
    codes = e2m1_encode(scaled, rounding).view(m, k)
    sf_b = ue4m3_byte(sf) if fmt == 'nvfp4' else ue8m0_byte(sf)
    return pack_nibbles(codes), sf, sf_b


def sf_bytes_to_float(sf_b: torch.Tensor, fmt: str) -> torch.Tensor:
    if fmt == 'nvfp4':
        return sf_b.view(torch.float8_e4m3fn).float()
    return (sf_b.to(torch.int32) << 23).view(torch.float32)


def dequant_fp4_rows(packed: torch.Tensor, sf: torch.Tensor, vec: int) -> torch.Tensor:
    """`dequant_fp4_rows` / `dequant_fp4` of `sm100_b200/test_mega_moe.py:94-98,414-419`."""
    vals = e2m1_decode(unpack_nibbles(packed))
    return vals * sf.repeat_interleave(vec, dim=-1)


def quant_fp8_rows(t: torch.Tensor, gran: int = 32, amax_floor: float = 1e-4,
                   sf_rule: str = 'div') -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[M, K] -> (e4m3 bytes uint8 [M, K], scale fp32 [M, K/32], UE8M0 bytes [M, K/32]).

    `per_token_cast_to_fp8(..., use_ue8m0=True, gran_k=32)` of
    `deep_gemm/utils/math.py:26-38`: amax clamped at 1e-4, scale
    2^ceil(log2(amax/448)), values `x * (1 / sf)` to E4M3.
    """
    m, k = t.shape
    g = t.float().view(m, k // gran, gran)
    amax = g.abs().amax(dim=-1).clamp_min(amax_floor)
    v = amax / 448.0 if sf_rule == 'div' else amax * torch.tensor(1.0 / 448.0, dtype=torch.float32)
    sf = ceil_pow2(v)
    q = (g * (1.0 / sf.unsqueeze(-1))).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(m, k)
    return q.view(torch.uint8), sf, ue8m0_byte(sf)


def dequant_fp8_rows(q_bytes: torch.Tensor, sf: torch.Tensor, gran: int = 32) -> torch.Tensor:
    """`dequant_fp8_ue8m0` of `sm100_b200/test_mega_moe.py:420-424`."""
    return q_bytes.view(torch.float8_e4m3fn).float() * sf.repeat_interleave(gran, dim=-1)


def requant_fp8_per32(a: torch.Tensor) -> torch.Tensor:
    """Intermediate requantisation of the FP8-activation kernel (`test_mega_moe.py:425-429`)."""
    if a.shape[0] == 0:
        return a
    g = a.view(a.shape[0], -1, 32)
    amax = g.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    sf = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    return ((g / sf).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * sf).view_as(a)


# ----------------------------------------------------------------------------- router
def router_reference(x: torch.Tensor, router_w: torch.Tensor, topk: int = 8,
                     score: str = 'softmax', bias: Optional[torch.Tensor] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """bf16 router GEMM (fp32 accumulate) -> bf16 logits -> top-k -> weights.

    `score='softmax'`: `tests/test_four_api_correctness.py:371-378` — stable
    descending sort of the bf16 logits (ties to the smaller expert id), fp32
    softmax over the selected logits, an all-zero token row gets idx -1 / w 0.
    -0.0 is canonicalised to +0.0 before the comparison
    (`sm100_b200/fe_sm100/fable_frontend_device.cuh:252-257`).
    `score='sigmoid_bias'` (benchmark configuration extension, not in the
    reference): scores = sigmoid(logit) + bias select the experts with the same
    tie rule; the weights are sigmoid(logit) of the selected experts renormalised
    to sum 1.
    Returns (topk_idx int64 [T, k], topk_weights fp32 [T, k], logits bf16 [T, E]).
    """
    logits = (x.float() @ router_w.float().t()).to(torch.bfloat16)
    lf = logits.float() + 0.0
    if score == 'softmax':
        order = torch.sort(lf, dim=-1, descending=True, stable=True).indices[:, :topk]
        sel = torch.gather(lf, 1, order)
        w = torch.softmax(sel, dim=-1)
    else:
        sig = torch.sigmoid(lf)
        sc = sig + (bias.float()[None, :] if bias is not None else 0.0)
        order = torch.sort(sc, dim=-1, descending=True, stable=True).indices[:, :topk]
        sel = torch.gather(sig, 1, order)
        w = sel / sel.sum(dim=-1, keepdim=True)
    idx = order.to(torch.int64)
    zero = (x.float() == 0).all(dim=-1)
    idx[zero] = -1
    w = w.clone()
    w[zero] = 0
    return idx, w.float(), logits


def balanced_routing(num_tokens: int, rank: int, num_ranks: int, num_experts: int, topk: int
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forced-balanced routing of `sm100_b200/test_mega_moe.py:113-123`.

    One rank: expert = (g * topk + s) % E. Several ranks: g = t + rank * 1000003,
    expert = r(s) * E_local + (g + 7 s) % E_local with weight 1/topk, where the
    reference (8 ranks, top-8) sends slot s to rank s; for fewer ranks than slots
    r(s) = s % num_ranks and the slots that share a rank are spread by adding
    (s // num_ranks) * 11 to the local index (extension, keeps a token's experts
    distinct).
    """
    s = torch.arange(topk, dtype=torch.int64)
    if num_ranks == 1:
        g = torch.arange(num_tokens, dtype=torch.int64)
        idx = (g[:, None] * topk + s[None, :]) % num_experts
    else:
        e_local = num_experts // num_ranks
        g = torch.arange(num_tokens, dtype=torch.int64) + rank * 1000003
        if num_ranks >= topk:
            idx = s[None, :] * e_local + (g[:, None] + 7 * s[None, :]) % e_local
        else:
            r = s % num_ranks
            idx = r[None, :] * e_local + (g[:, None] + 7 * s[None, :] + (s // num_ranks)[None, :] * 11) % e_local
    w = torch.full((num_tokens, topk), 1.0 / topk, dtype=torch.float32)
    return idx, w


# ----------------------------------------------------------------------------- the layer
@dataclass
class RankInput:
    """What one rank feeds the layer: quantised tokens and routing."""
    x_q: torch.Tensor            # packed E2M1 [T, H/2] uint8, or E4M3 bytes [T, H] for 'fp8'
    x_sf: torch.Tensor           # fp32 scales [T, H/vec]
    topk_idx: torch.Tensor       # int64 [T, k], -1 = masked
    topk_weights: torch.Tensor   # fp32 [T, k]


@dataclass
class RankWeights:
    """One rank's experts, untransformed: W1 rows [0, I) are gate, [I, 2I) up."""
    w1_q: torch.Tensor           # packed [E_local, 2I, H/2]
    w1_sf: torch.Tensor          # fp32 [E_local, 2I, H/vec_w]
    w2_q: torch.Tensor           # packed [E_local, H, I/2]
    w2_sf: torch.Tensor          # fp32 [E_local, H, I/vec_w]


@dataclass
class LayerResult:
    y: List[torch.Tensor]                     # per rank bf16 [T, H]
    counts: List[torch.Tensor]                # per rank int32 [E_local]: rows received per local expert
    slot_map: List[List[List[Tuple[int, int, int]]]]   # per rank, per local expert: [(src_rank, token, slot)] canonical order
    mid_q: List[Dict[int, torch.Tensor]] = field(default_factory=list)    # per rank {e_local: packed / e4m3 bytes [n, I(/2)]}
    mid_sf: List[Dict[int, torch.Tensor]] = field(default_factory=list)   # per rank {e_local: scale bytes [n, I/vec]}
    route_out: List[Dict[int, torch.Tensor]] = field(default_factory=list)  # per rank {e_local: bf16 [n, H]}


def canonical_slot_map(topk_idx_per_rank: Sequence[torch.Tensor], num_experts: int
                       ) -> List[List[List[Tuple[int, int, int]]]]:
    """Rows of a local expert ordered by (source rank, token, slot).

    The reference assigns pool rows by arrival-ordered tickets
    (`sm100_b200/sm100_fp4_fp4_mega_moe.cuh:533-560`), which no reference test
    observes; the per-expert counts are what its tests pin
    (`cumulative_local_expert_recv_stats`, `test_mega_moe.py:267-277`). This
    canonical order is this build's definition (parity of the order itself:
    unpinned in the reference).
    """
    num_ranks = len(topk_idx_per_rank)
    e_local = num_experts // num_ranks
    out = [[[] for _ in range(e_local)] for _ in range(num_ranks)]
    for src, idx in enumerate(topk_idx_per_rank):
        for t in range(idx.shape[0]):
            for s in range(idx.shape[1]):
                e = int(idx[t, s])
                if e >= 0:
                    out[e // e_local][e % e_local].append((src, t, s))
    return out


def swiglu_weighted(h: torch.Tensor, inter: int, clamp: Optional[float], w: torch.Tensor) -> torch.Tensor:
    """bf16-rounded gate/up, clamp, silu(gate) * up * topk weight (`test_mega_moe.py:456-459`)."""
    gate, up = h[:, :inter].to(torch.bfloat16), h[:, inter:].to(torch.bfloat16)
    if clamp is not None:
        gate = torch.clamp_max(gate, clamp)
        up = torch.clamp(up, -clamp, clamp)
    gate, up = gate.float(), up.float()
    return gate * torch.sigmoid(gate) * up * w[:, None]


def expert_forward(xs: torch.Tensor, ws: torch.Tensor, w1_q: torch.Tensor, w1_sf: torch.Tensor, w2_q: torch.Tensor,
                   w2_sf: torch.Tensor, act_format: str, clamp: Optional[float], rounding: str = 'rne',
                   w1_global_scale: float = 1.0, w2_global_scale: float = 1.0, mid_global_scale: float = 1.0,
                   dequantised: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """One expert on its routed rows (`sm100_b200/test_mega_moe.py:447-476`): dequantised `xs` [n, H] and top-k
    weights `ws` [n] -> (fp32 outputs [n, H], requantised intermediate, its scale bytes). `dequantised` = the
    expert's (W1, W2) already as fp32 (global scales applied) skips the weight dequantisation."""
    vec_a = SF_VEC[act_format]
    vec_w = 32 if act_format == 'fp8' else vec_a
    inter = w2_q.shape[-1] * 2
    if dequantised is not None:
        w1, w2 = dequantised
    else:
        w1 = dequant_fp4_rows(w1_q, w1_sf, vec_w) * w1_global_scale
        w2 = dequant_fp4_rows(w2_q, w2_sf, vec_w) * w2_global_scale
    act = swiglu_weighted(xs @ w1.t(), inter, clamp, ws)
    if act_format == 'fp8':
        q, sf, sfb = quant_fp8_rows(act, amax_floor=1e-30)
        mid = dequant_fp8_rows(q, sf)
    else:
        q, sf, sfb = quant_fp4_rows(act, act_format, rounding=rounding, sf_rule='div', global_scale=mid_global_scale)
        mid = dequant_fp4_rows(q, sf, vec_a) * mid_global_scale
    return mid @ w2.t(), q, sfb


def moe_rank_routes(inputs: Sequence[RankInput], local_experts: Dict[int, Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]],
                    rank: int, act_format: str, num_experts: int, clamp: Optional[float] = 10.0, rounding: str = 'rne',
                    x_global_scale: float = 1.0, w1_global_scale: float = 1.0, w2_global_scale: float = 1.0,
                    mid_global_scale: float = 1.0):
    """One rank's share of `moe_layer_reference` for a multi-process check (`sm100_b200/test_mega_moe.py:438-486`:
    every rank evaluates its own experts on the gathered tokens, then the partial results are all-reduced).

    `inputs`: all ranks' inputs; `local_experts`: {local expert id: (w1_q, w1_sf, w2_q, w2_sf)} for (at least) the
    experts of `rank` that receive rows. Returns ({(src rank, token, slot): bf16-rounded fp32 output row [H]},
    per-expert counts int32 [E_local], the canonical slot map of this rank)."""
    num_ranks = len(inputs)
    e_local = num_experts // num_ranks
    vec_a = SF_VEC[act_format]
    if act_format == 'fp8':
        x_dq = [dequant_fp8_rows(i.x_q, i.x_sf) for i in inputs]
    else:
        x_dq = [dequant_fp4_rows(i.x_q, i.x_sf, vec_a) * x_global_scale for i in inputs]
    smap = canonical_slot_map([i.topk_idx for i in inputs], num_experts)[rank]
    counts = torch.tensor([len(smap[e]) for e in range(e_local)], dtype=torch.int32)
    routes = {}
    for e in range(e_local):
        rows = smap[e]
        if not rows:
            continue
        xs = torch.stack([x_dq[src][t] for (src, t, s) in rows])
        ws = torch.stack([inputs[src].topk_weights[t, s] for (src, t, s) in rows]).float()
        out, _, _ = expert_forward(xs, ws, *local_experts[e], act_format, clamp, rounding, w1_global_scale,
                                   w2_global_scale, mid_global_scale)
        for n, key in enumerate(rows):
            routes[key] = out[n].to(torch.bfloat16).float()
    return routes, counts, smap


def moe_layer_reference(inputs: Sequence[RankInput], weights: Sequence[RankWeights], act_format: str,
                        num_experts: int, clamp: Optional[float] = 10.0, faithful: bool = True,
                        rounding: str = 'rne', keep_mid: bool = False,
                        x_global_scale: float = 1.0, w1_global_scale: float = 1.0,
                        w2_global_scale: float = 1.0, mid_global_scale: float = 1.0,
                        dequantised: Optional[Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]]] = None) -> LayerResult:
    """All ranks of the EP layer in one process (`sm100_b200/test_mega_moe.py:411-499`).

    Dequantised tokens and weights; per local expert an fp32 `X @ W1^T`, the
    SwiGLU with the top-k weight applied BEFORE the requantisation
    (`:459-460`), requantisation with the kernel's rule (`:425-437`), fp32
    `@ W2^T`, accumulation per token. The global scales (NVFP4 extension) multiply
    the dequantised operands; `mid_global_scale` divides the intermediate before
    its requantisation and multiplies it back after. `dequantised` optionally maps
    (rank, local expert) to that expert's (W1, W2) already dequantised to fp32
    (the reference dequantises all weights once, before its loop, `:411-420`).
    """
    num_ranks = len(inputs)
    e_local = num_experts // num_ranks
    vec_a = SF_VEC[act_format]
    vec_w = 32 if act_format == 'fp8' else vec_a
    hidden = weights[0].w1_q.shape[-1] * 2
    inter = weights[0].w2_q.shape[-1] * 2
    if act_format == 'fp8':
        x_dq = [dequant_fp8_rows(i.x_q, i.x_sf) for i in inputs]
    else:
        x_dq = [dequant_fp4_rows(i.x_q, i.x_sf, vec_a) * x_global_scale for i in inputs]
    smap = canonical_slot_map([i.topk_idx for i in inputs], num_experts)
    counts = [torch.tensor([len(smap[r][e]) for e in range(e_local)], dtype=torch.int32) for r in range(num_ranks)]
    acc = [[[None] * i.topk_idx.shape[1] for _ in range(i.topk_idx.shape[0])] for i in inputs]
    y32 = [torch.zeros((i.topk_idx.shape[0], hidden), dtype=torch.float32) for i in inputs]
    res = LayerResult(y=[], counts=counts, slot_map=smap)
    for r in range(num_ranks):
        mids, midsf, routes = {}, {}, {}
        for e in range(e_local):
            rows = smap[r][e]
            if not rows:
                continue
            xs = torch.stack([x_dq[src][t] for (src, t, s) in rows])
            ws = torch.stack([inputs[src].topk_weights[t, s] for (src, t, s) in rows]).float()
            out, q, sfb = expert_forward(xs, ws, weights[r].w1_q[e], weights[r].w1_sf[e], weights[r].w2_q[e],
                                         weights[r].w2_sf[e], act_format, clamp, rounding, w1_global_scale,
                                         w2_global_scale, mid_global_scale,
                                         dequantised.get((r, e)) if dequantised is not None else None)
            if keep_mid:
                mids[e], midsf[e] = q, sfb
                routes[e] = out.to(torch.bfloat16)
            for n, (src, t, s) in enumerate(rows):
                if faithful:
                    acc[src][t][s] = out[n].to(torch.bfloat16).float()
                else:
                    y32[src][t] += out[n]
        res.mid_q.append(mids)
        res.mid_sf.append(midsf)
        res.route_out.append(routes)
    for r, inp in enumerate(inputs):
        if faithful:
            for t in range(inp.topk_idx.shape[0]):
                for s in range(inp.topk_idx.shape[1]):
                    if acc[r][t][s] is not None:
                        y32[r][t] += acc[r][t][s]
        res.y.append(y32[r].to(torch.bfloat16))
    return res


# ----------------------------------------------------------------------------- synthetic workloads
def make_expert_weights(e_local: int, hidden: int, inter: int, fmt: str, seed: int, std: float = 0.02,
                        rounding: str = 'ref') -> Tuple[RankWeights, float, float]:
    """Seeded N(0, std) expert weights quantised per row like `cast_grouped_weights_to_fp4`
    (`sm100_b200/test_mega_moe.py:148-165`). For NVFP4 a per-tensor fp32 global scale
    amax / (6 * 448) is applied first (benchmark-configuration extension). Returns the
    weights and the two global scales (1.0 unless NVFP4).
    """
    g = torch.Generator().manual_seed(seed)
    wfmt = 'mxfp4' if fmt == 'fp8' else fmt
    w1 = (torch.randn((e_local, 2 * inter, hidden), generator=g) * std).to(torch.bfloat16)
    w2 = (torch.randn((e_local, hidden, inter), generator=g) * std).to(torch.bfloat16)
    gs1 = float(w1.float().abs().max() / (6.0 * 448.0)) if fmt == 'nvfp4' else 1.0
    gs2 = float(w2.float().abs().max() / (6.0 * 448.0)) if fmt == 'nvfp4' else 1.0
    q1, s1, q2, s2 = [], [], [], []
    for e in range(e_local):
        a, b, _ = quant_fp4_rows(w1[e], wfmt, rounding=rounding, global_scale=gs1)
        q1.append(a); s1.append(b)
        a, b, _ = quant_fp4_rows(w2[e], wfmt, rounding=rounding, global_scale=gs2)
        q2.append(a); s2.append(b)
    return RankWeights(torch.stack(q1), torch.stack(s1), torch.stack(q2), torch.stack(s2)), gs1, gs2


def quantise_tokens(x: torch.Tensor, fmt: str, rounding: str = 'rne', sf_rule: str = 'mul',
                    global_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Token quantisation as the frontend does it (`fable_frontend_sm100.cu:125-180`)."""
    if fmt == 'fp8':
        return quant_fp8_rows(x, sf_rule=sf_rule)
    return quant_fp4_rows(x, fmt, rounding=rounding, sf_rule=sf_rule, global_scale=global_scale)


def rel_rmse(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().flatten(), b.float().flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-30))


# ----------------------------------------------------------------------------- router, device reduction order
def router_logits_device_order(x: torch.Tensor, router_w: torch.Tensor) -> torch.Tensor:
    """bf16 router logits with the summation order of this build's frontend kernel, bit for bit.

    The reference's GEMV also fixes an order (fp32 FMA chain per lane, butterfly, K parts summed in order, one bf16
    rounding, `sm100_b200/fe_sm100/fable_frontend_sm100.cu:610-740`); its value-level contract is the torch rule of
    `router_reference`. Order used here: K is cut into two halves of ceil(K / 16) 8-element chunks; inside a half,
    lane l of 32 owns the chunks l, l + 32, ... and runs one fused multiply-add chain over them; the 32 partial sums
    are combined by a butterfly (xor 16, 8, 4, 2, 1); first half + second half in fp32; one rounding to bf16; -0.0
    becomes +0.0. The fused multiply-add is evaluated in float64 (the product of two bf16 values and the sum with an
    fp32 accumulator are exact there) and rounded once to fp32.
    """
    import numpy as np
    xf = x.float().numpy().astype(np.float64)
    wf = router_w.float().numpy().astype(np.float64)
    t, h = xf.shape
    e = wf.shape[0]
    nchunk = h // 8
    half = (nchunk + 1) // 2
    idx = np.arange(32)
    parts = []
    for c_lo in (0, half):
        c_hi = min(nchunk, c_lo + half)
        acc = np.zeros((t, e, 32), dtype=np.float32)
        for c0 in range(c_lo, c_hi, 32):
            lanes = min(32, c_hi - c0)
            for k in range(8):
                cols = (c0 + np.arange(lanes)) * 8 + k
                prod = xf[:, None, cols] * wf[None, :, cols]
                acc[:, :, :lanes] = (prod + acc[:, :, :lanes].astype(np.float64)).astype(np.float32)
        for o in (16, 8, 4, 2, 1):
            acc = (acc + acc[:, :, idx ^ o]).astype(np.float32)
        parts.append(acc[:, :, 0].copy())
    total = (parts[0] + parts[1]).astype(np.float32)
    logits = torch.from_numpy(total).to(torch.bfloat16)
    return (logits.float() + 0.0).to(torch.bfloat16)


def route_from_logits(logits: torch.Tensor, x: torch.Tensor, topk: int = 8, score: str = 'softmax',
                      bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k selection and weights from given bf16 logits (the rules of `router_reference`)."""
    lf = logits.float() + 0.0
    if score == 'softmax':
        order = torch.sort(lf, dim=-1, descending=True, stable=True).indices[:, :topk]
        w = torch.softmax(torch.gather(lf, 1, order), dim=-1)
    else:
        sig = torch.sigmoid(lf)
        sc = sig + (bias.float()[None, :] if bias is not None else 0.0)
        order = torch.sort(sc, dim=-1, descending=True, stable=True).indices[:, :topk]
        sel = torch.gather(sig, 1, order)
        w = sel / sel.sum(dim=-1, keepdim=True)
    idx = order.to(torch.int64)
    zero = (x.float() == 0).all(dim=-1)
    idx[zero] = -1
    w = w.clone().float()
    w[zero] = 0
    return idx, w
