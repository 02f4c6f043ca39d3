// Load-time preparation kernels: the pre-tiled weight stream (with the gate/up interleave and the scale-plane
// transposition folded in) and a row-wise E2M1 cast. Both are plain HBM copies with a little arithmetic on the way.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "mm_ptx.cuh"

namespace mm {

struct PrepParams {
    const uint8_t* w;                 // packed E2M1 [E][N][K/2], K-major, contiguous
    const void* sf;                   // int32 scale words (4 bytes = 4 consecutive K blocks) or fp32 scales
    long long sf_stride_e, sf_stride_n, sf_stride_k;   // in elements of the scale tensor's type
    int sf_is_fp32, E, N, K, vec, interleave;
    uint8_t* out;                     // [E][N/128][K/256][unit_bytes]
    uint32_t unit_bytes, planes;
};

// source row of output row n (L1: groups of 8 gate rows followed by the matching 8 up rows)
__device__ __forceinline__ uint32_t prep_source_row(uint32_t n, uint32_t N, int interleave) {
    if (!interleave) return n;
    const uint32_t g = n >> 4, w = n & 15u;
    return w < 8u ? g * 8u + w : N / 2u + g * 8u + (w - 8u);
}

// one scale byte from an fp32 scale: UE8M0 exponent (vec 32; non powers of two round up) or E4M3 (vec 16, RNE)
__device__ __forceinline__ uint32_t prep_sf_byte(float v, int vec) {
    if (vec == 16) return cvt_e4m3x2(v, 0.f) & 0xFFu;
    return ceil_pow2_exp(v);
}

// One CTA per streamed unit (expert, 128-row tile, 256-element K unit): 1024 16 B chunks of weights into the 128 B-swizzled
// image, then `planes` scale planes of 128 words in the (row % 32) * 4 + row / 32 order of the tensor-memory scale copy.
__global__ void __launch_bounds__(256) pretile_weights_kernel(const PrepParams q) {
    const uint32_t ku_n = q.K / 256u, nt_n = q.N / 128u;
    const uint32_t unit = blockIdx.x;
    const uint32_t ku = unit % ku_n, tile = (unit / ku_n) % nt_n, e = unit / (ku_n * nt_n);
    uint8_t* dst = q.out + static_cast<size_t>(unit) * q.unit_bytes;
    const size_t row_bytes = q.K / 2u;
    const uint8_t* wsrc = q.w + static_cast<size_t>(e) * q.N * row_bytes;
    uint4 v[4];
    #pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t idx = i * 256u + threadIdx.x, r = idx >> 3, ch = idx & 7u;
        const uint32_t src_row = prep_source_row(tile * 128u + r, q.N, q.interleave);
        v[i] = ld_cg_v4(wsrc + static_cast<size_t>(src_row) * row_bytes + ku * 128u + ch * 16u);
    }
    #pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t idx = i * 256u + threadIdx.x, r = idx >> 3, ch = idx & 7u;
        *reinterpret_cast<uint4*>(dst + r * 128u + ((ch ^ (r & 7u)) << 4)) = v[i];
    }
    for (uint32_t idx = threadIdx.x; idx < 128u * q.planes; idx += 256u) {
        const uint32_t pl = idx >> 7, r = idx & 127u;
        const uint32_t src_row = prep_source_row(tile * 128u + r, q.N, q.interleave);
        const uint32_t word_k = ku * q.planes + pl;                        // scale word index along K (4 scale bytes each)
        uint32_t word;
        if (q.sf_is_fp32) {
            const float* s = static_cast<const float*>(q.sf) + e * q.sf_stride_e + static_cast<long long>(src_row) * q.sf_stride_n;
            word = 0u;
            #pragma unroll
            for (uint32_t b = 0; b < 4; ++b) word |= prep_sf_byte(s[(word_k * 4u + b) * q.sf_stride_k], q.vec) << (8u * b);
        } else {
            word = static_cast<const uint32_t*>(q.sf)[e * q.sf_stride_e + static_cast<long long>(src_row) * q.sf_stride_n + word_k * q.sf_stride_k];
        }
        reinterpret_cast<uint32_t*>(dst + 16384u + pl * 512u)[(r & 31u) * 4u + (r >> 5)] = word;
    }
}

// Row-wise cast to packed E2M1 with one scale per `gran` elements, the arithmetic of the reference's host helper:
// block maximum clamped at 1e-4, scale = amax / 6 (rounded up to a power of two when `ue8m0`), x * (1 / scale), codes by
// the midpoint comparisons 0.25 / 0.75 / 1.25 / 1.75 / 2.5 / 3.5 / 5 with ties toward the smaller magnitude, sign bit only
// on non-zero codes. One thread per 8 elements; the `gran / 8` threads of a block share the maximum by shuffles.
template <typename T>
__global__ void __launch_bounds__(256) cast_rows_fp4_kernel(const T* __restrict__ x, int M, int K, int gran, int ue8m0,
                                                            uint8_t* __restrict__ packed, float* __restrict__ sf) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long per_row = K / 8;
    const bool live = t < static_cast<long long>(M) * per_row;
    const long long row = live ? t / per_row : 0, c8 = live ? t % per_row : 0;
    float v[8];
    #pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = live ? static_cast<float>(x[row * K + c8 * 8 + j]) : 0.f;
    float amax = 0.f;
    #pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    for (int o = 1; o < gran / 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float s = __fdiv_rn(fmaxf(amax, 1e-4f), 6.0f);
    if (ue8m0) s = __uint_as_float(ceil_pow2_exp(s) << 23);
    const float inv = __fdiv_rn(1.0f, s);
    uint32_t out = 0u;
    #pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float a = fabsf(v[j] * inv);
        uint32_t code = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
        if (v[j] * inv < 0.f && code != 0u) code |= 8u;
        out |= code << (4 * j);
    }
    if (live) {
        *reinterpret_cast<uint32_t*>(packed + row * (K / 2) + c8 * 4) = out;
        if ((c8 % (gran / 8)) == 0) sf[row * (K / gran) + c8 / (gran / 8)] = s;
    }
}

// Largest magnitude of a tensor (grid-stride, 16 B loads, one atomic per block): the calibration step of a per-tensor
// global scale. `out` holds the bit pattern of a non-negative float (such patterns order like unsigned integers) and must
// start at zero; NaNs are ignored.
template <typename T>
__global__ void __launch_bounds__(256) absmax_kernel(const T* __restrict__ x, long long n, uint32_t* __restrict__ out) {
    constexpr int kPer = 16 / sizeof(T);
    float m = 0.f;
    const long long nvec = n / kPer;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const uint4 q = ld_cg_v4(reinterpret_cast<const uint4*>(x) + i);
        const T* v = reinterpret_cast<const T*>(&q);
        #pragma unroll
        for (int j = 0; j < kPer; ++j) m = fmaxf(m, fabsf(static_cast<float>(v[j])));
    }
    if (blockIdx.x == 0 && threadIdx.x < n - nvec * kPer) m = fmaxf(m, fabsf(static_cast<float>(x[nvec * kPer + threadIdx.x])));
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        #pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, part[w]);
        atomicMax(out, __float_as_uint(m));
    }
}

}  // namespace mm
