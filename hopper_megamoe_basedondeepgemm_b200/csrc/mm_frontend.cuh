// Router frontend: bf16 router GEMM (fp32 accumulate, one bf16 rounding), top-8 selection with the
// (score descending, expert id ascending) order, routing weights, and token quantisation into the layer's input views.
//
// Reduction order of a logit (fixed, so that a CPU restatement can reproduce it bit for bit): K is cut into two halves;
// inside a half, lane l of a warp owns the 8-element chunks l, l + 32, l + 64, ... and runs one fused multiply-add chain
// over them in order; the 32 partial sums are combined by a butterfly (xor 16, 8, 4, 2, 1); the two halves are added
// (first + second) in fp32 and the sum is rounded to bf16 once. A half is one warp's work with all its loads in flight
// at once: one memory round trip per logit.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "mm_ptx.cuh"

namespace mm {

struct FeParams {
    const __nv_bfloat16* hidden; const __nv_bfloat16* router_w; const float* bias;
    float* logits; uint32_t* arrive;
    uint8_t* x; uint8_t* x_sf; long long* topk_idx; float* topk_w;
    int T, H, E, topk, score_mode, fmt, x_row_bytes, x_sf_row_bytes;
    float x_gs;
};

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}

constexpr uint32_t kFeParts = 2;
constexpr int kFeMaxFusedTokens = 256;       // tokens per rank the single-kernel path takes (its logit records live in the buffer)

// Partial logits live in the workspace as 16 B records per (token, expert): {first half, flag, second half, flag}; each
// half is written by its warp with one 8-byte store, so a reader that finds `flag` in a half also has its value.
// One warp per (expert, half of K, block of up to 4 tokens); `warp` of `nwarps` warps cooperate.
__device__ __forceinline__ void fe_logits_items(const FeParams& q, uint32_t warp, uint32_t nwarps, uint32_t lane, uint32_t flag) {
    const uint32_t tblocks = (q.T + 3) / 4, nchunk = q.H / 8, half = (nchunk + kFeParts - 1) / kFeParts;
    const uint32_t nitems = static_cast<uint32_t>(q.E) * kFeParts * tblocks;
    for (uint32_t item = warp; item < nitems; item += nwarps) {
        const uint32_t part = item % kFeParts, e = (item / kFeParts) % q.E, t0 = (item / (kFeParts * q.E)) * 4;
        const uint32_t nt = min(4u, static_cast<uint32_t>(q.T) - t0);
        const uint32_t c_lo = part * half, c_hi = min(nchunk, c_lo + half);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const uint4* wrow = reinterpret_cast<const uint4*>(q.router_w + static_cast<size_t>(e) * q.H);
        // six chunks per lane are fetched before the first multiply-add (a half of K = 3072 is exactly that: one memory
        // round trip); the multiply-adds then run in the same order as a chunk-by-chunk loop would
        constexpr uint32_t kAhead = 6;
        #pragma unroll 1
        for (uint32_t ch0 = c_lo + lane; ch0 < c_hi; ch0 += 32 * kAhead) {
            uint4 wq[kAhead], xq[4][kAhead];
            #pragma unroll
            for (uint32_t b = 0; b < kAhead; ++b) {
                const uint32_t ch = ch0 + 32 * b;
                if (ch < c_hi) {
                    wq[b] = __ldg(wrow + ch);
                    #pragma unroll
                    for (uint32_t t = 0; t < 4; ++t)
                        if (t < nt) xq[t][b] = __ldg(reinterpret_cast<const uint4*>(q.hidden + static_cast<size_t>(t0 + t) * q.H) + ch);
                }
            }
            #pragma unroll
            for (uint32_t b = 0; b < kAhead; ++b) {
                if (ch0 + 32 * b < c_hi) {
                    float w[8];
                    unpack_bf16x8(wq[b], w);
                    #pragma unroll
                    for (uint32_t t = 0; t < 4; ++t) {
                        if (t < nt) {
                            float x[8];
                            unpack_bf16x8(xq[t][b], x);
                            #pragma unroll
                            for (int k = 0; k < 8; ++k) acc[t] = fmaf(x[k], w[k], acc[t]);
                        }
                    }
                }
            }
        }
        #pragma unroll
        for (uint32_t t = 0; t < 4; ++t) {
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
            if (lane == 0 && t < nt)
                st_volatile_v2(reinterpret_cast<uint8_t*>(q.logits) + (static_cast<size_t>(t0 + t) * q.E + e) * 16u + part * 8u,
                               __float_as_uint(acc[t]), flag);
        }
    }
}

// logit of (token t, expert e) from its two halves; `flag` != 0: poll until both halves carry it (`ok` = false if `give_up`
// says so first)
template <typename GiveUp>
__device__ __forceinline__ float fe_read_logit(const FeParams& q, uint32_t t, uint32_t e, uint32_t flag, bool& ok, GiveUp give_up) {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(q.logits) + (static_cast<size_t>(t) * q.E + e) * 16u;
    uint32_t spins = 0;
    for (;;) {
        const uint4 v = ld_volatile_v4(src);
        if (flag == 0u || (v.y == flag && v.w == flag)) return bf16_round(__uint_as_float(v.x) + __uint_as_float(v.z)) + 0.0f;
        if ((++spins & 0x3Fu) == 0u && give_up()) { ok = false; return 0.f; }
    }
}

__global__ void __launch_bounds__(256) frontend_logits_kernel(const FeParams q) {
    fe_logits_items(q, blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), gridDim.x * (blockDim.x >> 5), threadIdx.x & 31u, 1u);
}

__device__ __forceinline__ uint32_t orderable_f32(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    return v;
}

// One warp quantises token row `xrow` (bf16 [H]) to packed E2M1 (formats 0, 1) or E4M3 bytes (format 2) + scale bytes;
// returns whether any element is non-zero. With `pool_row` != nullptr the same bytes are also stored there as a row of
// the receive pool (packed row, then the scale bytes; every 4 data bytes followed by `flag`): the dispatch of the fused
// frontend writes the peer's pool straight from the registers instead of re-reading the views it has just written.
__device__ __forceinline__ bool fe_quant_token(const __nv_bfloat16* xrow, int H, int fmt, float x_gs,
                                               uint8_t* qrow, uint8_t* sfrow, uint32_t lane,
                                               uint8_t* pool_row = nullptr, uint32_t flag = 0u, uint32_t x_row_bytes = 0u) {
    const int vec = fmt == 1 ? 16 : 32, lanes_per_group = vec / 8;
    bool nonzero = false;
    for (int k0 = lane * 8; k0 < H; k0 += 256) {
        float x[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(xrow + k0), x);
        float local = 0.f;
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            nonzero |= x[j] != 0.f;
            if (fmt == 1) x[j] = __fdiv_rn(x[j], x_gs);
            local = fmaxf(local, fabsf(x[j]));
        }
        local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, 1));
        if (lanes_per_group == 4) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, 2));
        const float v = fmt == 2 ? fmaxf(local, 1.0e-4f) * (1.0f / 448.0f) : fmaxf(local, 1.0e-30f) * (1.0f / 6.0f);
        uint32_t sf_byte; float sf;
        if (fmt == 1) {
            sf_byte = cvt_e4m3x2(v, 0.f) & 0xFFu;
            if (sf_byte == 0u) sf_byte = 1u;
            sf = e4m3_to_float(sf_byte);
        } else {
            sf_byte = ceil_pow2_exp(v);
            sf = __uint_as_float(sf_byte << 23);
        }
        if ((lane % lanes_per_group) == 0) sfrow[k0 / vec] = static_cast<uint8_t>(sf_byte);
        const float inv = 1.0f / sf;
        const int it = k0 >> 8;                                  // which 256-element slice of the row
        if (fmt == 2) {
            uint2 bytes;
            bytes.x = cvt_e4m3x2(x[0] * inv, x[1] * inv) | (cvt_e4m3x2(x[2] * inv, x[3] * inv) << 16);
            bytes.y = cvt_e4m3x2(x[4] * inv, x[5] * inv) | (cvt_e4m3x2(x[6] * inv, x[7] * inv) << 16);
            *reinterpret_cast<uint2*>(qrow + k0) = bytes;
            if (pool_row != nullptr) {
                asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" :: "l"(pool_row + 2 * k0), "r"(bytes.x), "r"(flag), "r"(bytes.y), "r"(flag) : "memory");
            }
        } else {
            uint32_t packed = 0u;
            #pragma unroll
            for (int j = 0; j < 4; ++j) packed |= cvt_e2m1x2(x[2 * j] * inv, x[2 * j + 1] * inv) << (8 * j);
            *reinterpret_cast<uint32_t*>(qrow + k0 / 2) = packed;
            if (pool_row != nullptr) st_volatile_v2(pool_row + k0, packed, flag);          // 2 * (k0 / 2)
        }
        if (pool_row != nullptr) {
            // four scale bytes make one word: every lane of a group holds its group's byte; the first lane of four groups stores
            const int span = 4 * lanes_per_group;               // lanes that share one scale word
            const uint32_t base_lane = lane & ~static_cast<uint32_t>(span - 1);
            uint32_t word = 0u;
            #pragma unroll
            for (int b = 0; b < 4; ++b) word |= __shfl_sync(0xffffffffu, sf_byte, base_lane + b * lanes_per_group) << (8 * b);
            if ((lane & static_cast<uint32_t>(span - 1)) == 0u) {
                const uint32_t sf_off = static_cast<uint32_t>(it) * (256u / vec) + (lane / span) * 4u;     // byte offset inside the row's scale bytes
                st_volatile_v2(pool_row + 2u * (x_row_bytes + sf_off), word, flag);
            }
        }
    }
    return __any_sync(0xffffffffu, nonzero);
}

// One warp: is any element of the bf16 row non-zero?
__device__ __forceinline__ bool fe_row_nonzero(const __nv_bfloat16* xrow, int H, uint32_t lane) {
    // all loads of the row are issued before the first is used (one memory round trip, not one per 256 elements); the
    // row then sits in this SM's L1 for the quantisation pass that follows with the same lane mapping
    uint32_t any = 0u;
    #pragma unroll
    for (int i = 0; i < 16; ++i) {                        // H <= 4096
        const int k0 = lane * 8 + i * 256;
        if (k0 < H) {
            const uint4 v = *reinterpret_cast<const uint4*>(xrow + k0);
            any |= v.x | v.y | v.z | v.w;
        }
    }
    const bool nz = (any & 0x7FFF7FFFu) != 0u;
    return __any_sync(0xffffffffu, nz);
}

// One warp selects the top-8 experts of token t from its logits (other SMs wrote them; `flag` != 0: they may still be on
// their way and are polled) and writes topk_idx / topk_weights. `sc` is a per-warp scratch of 2 E floats in shared
// memory (scores, then the plain logits). Returns false if `give_up` ended a poll.
template <typename GiveUp>
__device__ __forceinline__ bool fe_select_token(const FeParams& q, uint32_t t, float* sc, bool nonzero, uint32_t lane, uint32_t flag, GiveUp give_up) {
    float* lgv = sc + q.E;
    bool ok = true;
    // the token's logit records, eight per lane in flight at a time (one memory round trip per 256 experts when they have
    // all arrived); a record that is not complete yet is polled on its own afterwards
    for (int e0 = lane; e0 < q.E; e0 += 32 * 8) {
        uint4 rec[8];
        #pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int e = e0 + 32 * b;
            if (e < q.E) rec[b] = ld_volatile_v4(reinterpret_cast<const uint8_t*>(q.logits) + (static_cast<size_t>(t) * q.E + e) * 16u);
        }
        #pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int e = e0 + 32 * b;
            if (e >= q.E) continue;
            float v;
            if (flag == 0u || (rec[b].y == flag && rec[b].w == flag)) v = bf16_round(__uint_as_float(rec[b].x) + __uint_as_float(rec[b].z)) + 0.0f;
            else v = fe_read_logit(q, t, static_cast<uint32_t>(e), flag, ok, give_up);
            lgv[e] = v;
            sc[e] = q.score_mode == 1 ? (1.0f / (1.0f + expf(-v))) + q.bias[e] : v;
        }
    }
    if (!__all_sync(0xffffffffu, ok)) return false;
    __syncwarp();
    // eight rounds of a warp-wide maximum over 64-bit keys (score, then smaller expert id)
    unsigned long long chosen = 0ull;
    for (int k = 0; k < 8; ++k) {
        unsigned long long best = 0ull;
        for (int e = lane; e < q.E; e += 32) {
            const float s = sc[e];
            if (s == -INFINITY) continue;
            const unsigned long long key = (static_cast<unsigned long long>(orderable_f32(s + 0.0f)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(e));
            best = key > best ? key : best;
        }
        best = warp_max_u64(best);
        // no candidate left (fewer than eight selectable experts: every remaining score is -inf): the slot stays empty
        const bool found = best != 0ull;
        const uint32_t e_best = 0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFull);
        if (found && lane == 0) sc[e_best] = -INFINITY;
        if (static_cast<int>(lane) == k) chosen = found ? e_best : 0xFFFFFFFFull;
        __syncwarp();
    }
    const bool empty_slot = lane < 8 && chosen == 0xFFFFFFFFull;
    const int e_sel = empty_slot ? 0 : static_cast<int>(chosen);
    const float v_sel = lane < 8 && !empty_slot ? lgv[e_sel] : -INFINITY;
    float wgt;
    if (q.score_mode == 1) {
        const float s = lane < 8 ? 1.0f / (1.0f + expf(-v_sel)) : 0.f;
        float sum = 0.f;
        #pragma unroll
        for (int k = 0; k < 8; ++k) sum += __shfl_sync(0xffffffffu, s, k);
        wgt = s / sum;
    } else {
        float mx = v_sel;
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float ex = lane < 8 ? expf(v_sel - mx) : 0.f;
        float sum = 0.f;
        #pragma unroll
        for (int k = 0; k < 8; ++k) sum += __shfl_sync(0xffffffffu, ex, k);
        wgt = ex / sum;
    }
    if (lane < 8) {
        q.topk_idx[static_cast<size_t>(t) * 8 + lane] = nonzero && !empty_slot ? e_sel : -1;
        q.topk_w[static_cast<size_t>(t) * 8 + lane] = nonzero && !empty_slot ? wgt : 0.f;
    }
    return true;
}

// one warp per token: the token's quantisation, then top-8 + weights
__global__ void __launch_bounds__(128) frontend_select_quant_kernel(const FeParams q) {
    extern __shared__ float fe_scores[];                 // [4 warps][2 E]
    const uint32_t lane = threadIdx.x & 31u, w = threadIdx.x >> 5;
    const uint32_t t = blockIdx.x * 4 + w;
    if (t >= static_cast<uint32_t>(q.T)) return;
    const bool nonzero = fe_quant_token(q.hidden + static_cast<size_t>(t) * q.H, q.H, q.fmt, q.x_gs,
                                        q.x + static_cast<size_t>(t) * q.x_row_bytes, q.x_sf + static_cast<size_t>(t) * q.x_sf_row_bytes, lane);
    fe_select_token(q, t, fe_scores + w * 2 * q.E, nonzero, lane, 0u, [] { return false; });
}

}  // namespace mm
