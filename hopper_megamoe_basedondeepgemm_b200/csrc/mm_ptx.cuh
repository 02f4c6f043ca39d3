// Raw PTX wrappers for sm_100a: mbarrier, bulk async copies, tcgen05 (TMEM, UMMA, UTCCP),
// scoped loads/stores for the cross-CTA and cross-GPU counters. No CUTLASS dependency.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>

namespace mm {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t) :: "memory");
    return t;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 r;\n\t"
        "elect.sync r|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// ----------------------------------------------------------------------------- bulk async copy (TMA, untiled)
// global -> shared, completion counted in bytes on an mbarrier. Both addresses 16 B aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void prefetch_l2_line(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// global -> L2 only (no shared-memory destination, no completion to wait for). Address 16 B aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
// generic-proxy shared-memory writes -> visible to the async proxy (UMMA / UTCCP / bulk copies)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------- named barriers
// orders this thread's earlier accesses through the generic proxy (plain loads, stores, acquires) with its later
// asynchronous-proxy operations (bulk copies) and the other way round, in every state space
__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// counts the calling warp in on a named barrier without waiting for it
__device__ __forceinline__ void bar_arrive(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// barrier + OR-reduction of a predicate over the participating threads: every participant gets the same answer
__device__ __forceinline__ bool bar_red_or(uint32_t id, uint32_t nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"(static_cast<uint32_t>(pred)), "r"(id), "r"(nthreads) : "memory");
    return r != 0u;
}

// ----------------------------------------------------------------------------- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// all previously issued tcgen05 async ops of this thread -> one arrival on the mbarrier when they complete
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptor (sm_100 format): start address >> 4 in bits [0,14), leading byte offset >> 4 in
// [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), layout type in [61,64) (0 none, 2 = 128 B swizzle)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t layout_type) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= static_cast<uint64_t>(layout_type & 7) << 61;
    return d;
}
constexpr uint32_t kLayoutNone = 0, kLayoutSw128 = 2;

// block-scaled instruction descriptor: B scale id [4,6), A format [7,10), B format [10,13), N >> 3 in [17,23),
// scale format bit 23 (0 UE4M3, 1 UE8M0), M >> 4 in [24,29), A scale id [29,31). K-major operands, no negation.
__host__ __device__ constexpr uint32_t idesc_block_scaled(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n, uint32_t ue8m0) {
    return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (ue8m0 << 23) | ((m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf(uint32_t base, uint32_t a_sf_id, uint32_t b_sf_id) {
    return base | (b_sf_id << 4) | (a_sf_id << 29);
}
constexpr uint32_t kFmtMxf4E2M1 = 1;   // kind::mxf4 / kind::mxf4nvf4 operand format
constexpr uint32_t kFmtF8E4M3 = 0, kFmtF8E2M1 = 5;   // kind::mxf8f6f4 operand formats

// 32 lanes x 128 bit from shared memory into TMEM, replicated to the four 32-lane quarters
__device__ __forceinline__ void utccp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], E2M1 operands, UE8M0 scale per 32 elements, K = 64 per instruction
__device__ __forceinline__ void umma_mxf4_block32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// same with UE4M3 scale per 16 elements (NVFP4)
__device__ __forceinline__ void umma_nvf4_block16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// 8-bit containers (E4M3 activations x E2M1 weights), UE8M0 scale per 32 elements, K = 32 per instruction
__device__ __forceinline__ void umma_mxf8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}

// ----------------------------------------------------------------------------- scoped memory operations
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_volatile_u64(const void* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_acq_rel_gpu_add(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
// Flagged 8-byte words ("LL" lines): a 16 B store carries two {data, flag} pairs; each 8-byte half is written
// atomically, so a reader that sees the expected flag in a pair also sees that pair's data. No fence, no separate
// completion flag: one NVLink one-way trip from the store to the consumer.
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_ll_16B(void* dst, uint4 data, uint32_t flag) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" :: "l"(dst), "r"(data.x), "r"(flag), "r"(data.y), "r"(flag) : "memory");
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" :: "l"(static_cast<uint8_t*>(dst) + 16), "r"(data.z), "r"(flag), "r"(data.w), "r"(flag) : "memory");
}
// One 16 B half of a flagged 32 B chunk: half 0 carries payload words x, y, half 1 words z, w. Two neighbouring lanes
// that store the two halves of a chunk write one full 32 B sector with one instruction; a lane that stores both halves
// itself (st_ll_16B) touches every sector twice, half at a time, which costs twice the packets on NVLink.
__device__ __forceinline__ void st_ll_half(void* chunk_dst, const uint4& data, uint32_t flag, uint32_t half) {
    const uint32_t a = half ? data.z : data.x, b = half ? data.w : data.y;
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" :: "l"(static_cast<uint8_t*>(chunk_dst) + half * 16u), "r"(a), "r"(flag), "r"(b), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t data, uint32_t flag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" :: "l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ bool ll_valid(const uint4& a, const uint4& b, uint32_t flag) {
    return a.y == flag && a.w == flag && b.y == flag && b.w == flag;
}
__device__ __forceinline__ uint4 ll_data(const uint4& a, const uint4& b) { return make_uint4(a.x, a.z, b.x, b.z); }

__device__ __forceinline__ void st_global_v4(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ----------------------------------------------------------------------------- small integer division
// a / b for a < 2^24, b > 0 and a / b < 2^21 (tile, unit, SM, token and chunk indices are far below that) through one
// approximate float division (2 ulp) and a +-1 correction: about a dozen instructions
// instead of the ~100-cycle integer division sequence (these sit on per-unit and per-launch critical paths).
__device__ __forceinline__ uint32_t udiv_small(uint32_t a, uint32_t b) {
    uint32_t q = __float2uint_rz(__fdividef(static_cast<float>(a), static_cast<float>(b)));
    const int32_t r = static_cast<int32_t>(a - q * b);
    if (r < 0) --q; else if (static_cast<uint32_t>(r) >= b) ++q;
    return q;
}

// ----------------------------------------------------------------------------- numeric conversions
// two floats -> one byte of two E2M1 codes (round to nearest even, saturating); `lo` lands in the low nibble
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t d;
    asm("{ .reg .b8 b0; cvt.rn.satfinite.e2m1x2.f32 b0, %1, %2; cvt.u16.u8 %0, b0; }" : "=h"(d) : "f"(hi), "f"(lo));
    return static_cast<uint32_t>(d & 0xFFu);
}
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
    return static_cast<uint32_t>(d);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    uint32_t h2;
    uint16_t in = static_cast<uint16_t>(byte & 0xFFu);
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFFu)));
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// 2^ceil(log2(v)) from the float bits, exponent clamped to [1, 254]; returns the exponent byte
__device__ __forceinline__ uint32_t ceil_pow2_exp(float v) {
    const uint32_t bits = __float_as_uint(v);
    uint32_t ex = ((bits >> 23) & 0xFFu) + ((bits & 0x7FFFFFu) != 0u ? 1u : 0u);
    return ex < 1u ? 1u : (ex > 254u ? 254u : ex);
}

}  // namespace mm
