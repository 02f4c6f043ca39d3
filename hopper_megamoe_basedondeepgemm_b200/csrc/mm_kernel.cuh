// The fused expert-parallel MoE layer as one persistent sm_100a kernel.
//
//   dispatch  : SM d (< ranks) packs this rank's routed rows for rank d and stores them, densely and in (token, slot)
//               order, into a region of rank d's receive pool that only this rank writes. Everything that crosses
//               NVLink travels as flagged 8-byte words {4 data bytes, launch number}: the consumer polls the words it
//               needs, so there is no fence, no completion flag and no ticket atomic - one one-way trip per hand-off.
//   schedule  : every SM reads the R header lines, scans the received rows' records and derives its own task list in closed
//               form (L1 tiles of all active experts, then L2 tiles). A phase's NT tiles are split in two: each of the
//               first NT % SMs tiles is cut along K between the SMs of a fixed group (partial sums parked in global
//               memory, summed in SM order by the last contributor); the rest are whole tiles dealt round-robin.
//   L1 GEMM   : 128 weight rows x 16 tokens per task, swap-AB block-scaled tcgen05 MMA, accumulators in TMEM. Weights
//               arrive as pre-tiled 128 B-swizzled units with their scale planes by one bulk async copy per stage.
//               FP8-activation variant: eight more warps widen every packed unit to byte-wide operand slots in shared
//               memory (kind::mxf8f6f4 reads 4-bit values from 8-bit containers); HBM still streams the packed form.
//   L1 epilog : SwiGLU * top-k weight, requantise to E2M1 or E4M3 (+ scale byte), store to the local intermediate
//               pool as flagged words.
//   L2 GEMM   : the stager polls the intermediate rows it needs, same main loop on W2, epilogue stores bf16 rows
//               (flagged words) straight into the source rank's combine buffer over NVLink.
//   combine   : each thread polls the flagged words of the routes it sums; routes are added in slot order (fp32) and
//               written to y. No grid-wide or cross-rank barrier anywhere in the launch.
//
// Every wait is bounded by a deadline; on expiry the SM records a status word, raises a CTA-wide abort flag and all
// roles fall through to the common exit (TMEM is always released).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include "mm_ptx.cuh"
#include "mm_frontend.cuh"

namespace mm {

constexpr int kThreads = 256;
constexpr int kMaxRanks = 8;
constexpr int kMaxLocalExperts = 64;
constexpr int kMaxTasks = 256;          // tasks one SM can own in one launch
constexpr int kMetaCap = 4096;          // rows one rank can receive in one launch
constexpr int kMaxStages = 12;
constexpr int kDefaultStages = 4;       // stages used when shared memory allows more (see the launch code)
constexpr int kMetaSmemRows = 128;      // received rows whose (token, slot, weight) records are cached in shared memory
constexpr int kMaxMTiles = kMetaCap / 16 + kMaxLocalExperts;   // 16-token tiles over all local experts
constexpr int kTileRows = 128;          // UMMA M: weight rows per task
constexpr int kTileTokens = 16;         // UMMA N: token rows per task
constexpr int kUnitK = 256;             // K elements per streamed unit (one 128 B swizzle atom of packed E2M1)
constexpr int kUnitWBytes = kTileRows * 128;
constexpr int kNumEpiThreads = 128;
constexpr uint32_t kBarEpi = 1;          // named barrier of the four epilogue warps
constexpr uint32_t kBarCopy = 2;         // named barrier of the warps that dispatch
// The scout warp runs beside the other warps of the CTA from kernel entry to the start of the roles; it meets them at
// four named barriers, each used once per launch: kBarPrologue (the scout arrives without waiting, the others wait),
// kBarOwn (the scout arrives when its list of own rows is written; the others wait for it), kBarGo (the others arrive
// after the prologue; the scout waits before it uses the launch number), kBarSched (the others arrive when the task
// list is written; the scout waits, then takes up its role). kBarMain synchronises the other warps among themselves;
// after the received rows' records are scanned, only warps 0 and 1 go on to the schedule (kBarPost is theirs) and arrive
// on kBarSched, where all other warps wait.
constexpr uint32_t kBarOwn = 3, kBarGo = 4, kBarSched = 5, kBarMain = 6, kBarPrologue = 7, kBarPost = 8;
constexpr int kNumExpThreads = 256;      // FP8-activation variant: warps 8..15 widen the packed E2M1 weights to 8-bit containers
constexpr uint32_t kXbufBytes = 2 * kUnitWBytes + 1024;   // one widened unit + its two scale planes
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kFillWarps = 5;       // warps 2..6 fetch the received rows into shared memory while the schedule is built
constexpr uint32_t kOtileBytes = 8192;
constexpr uint32_t kMaxRecSlots = 8;      // slots of the token-record ring
constexpr uint32_t kRelQueue = 8;         // entries of the epilogue -> releasing warp queue
constexpr uint32_t kWideTokens = 32;      // token tile of the launches whose experts have more than 16 rows
constexpr uint32_t kVtStride = kTileRows + 8;   // floats between the tokens of the accumulator tile (tile-image epilogue: conflict-free 16 B reads)
constexpr uint32_t kVtBytes = kWideTokens * kVtStride * 4;   // fp32 accumulators of one task, token-major

constexpr int kOwnCap = 128;            // routed rows of this rank's own tokens that every SM lists for itself (see the scout)

// control-block offsets (bytes from off_ctrl)
constexpr int kCtrlEpoch = 0;           // u32[256] one launch counter per SM
constexpr int kCtrlStatus = 1024;       // u32[16]
constexpr int kCtrlStamps = 2048;       // u64[32] phase stamps
constexpr int kCtrlSmEntry = 4096;      // u64[256] per-SM time of the kernel's first instruction
constexpr int kCtrlSmWFirst = 6144;     // u64[256] per-SM time of the first weight request (prefetch or load); ~0: none
constexpr int kSmPhaseSlots = 32;       // per SM: 16 phase times, then the landing times of its first 16 weight units
constexpr int kCtrlSmPhase = 8192;      // u64[256][kSmPhaseSlots] per-SM phase times (see SmPhase)
constexpr int kCtrlBytes = 8192 + 256 * kSmPhaseSlots * 8;

// tuning bits (KParams::knobs)
enum : uint32_t {
    kKnobPrefetch = 1u,                 // the scout asks for the weights of every expert it learns to be live (L2 prefetch)
    kKnobOwnRows = 2u,                  // rows of this rank's own tokens are listed from topk_idx by every SM (no header wait)
    kKnobEarlyCombine = 4u,             // warps start on the combine as soon as their role ends
    kKnobRehearse = 8u,                 // idle role warps run their code once on made-up tasks before the roles start
    kKnobWaitProfile = 32u,             // the roles add up the cycles they spend waiting; totals replace the per-unit landing times in the SM records
    kKnobTileImages = 16u               // launches with more than 16 received rows: operand tiles prepared in global memory, fetched by bulk copies
};

// device status codes (low byte of status word 0)
enum : uint32_t {
    kErrWaitEmpty = 1, kErrWaitFull = 2, kErrWaitActsFull = 3, kErrWaitActsEmpty = 4, kErrWaitTmemFull = 5,
    kErrWaitTmemEmpty = 6, kErrWaitDispatchFlag = 7 /* header line or row words of a source rank */, kErrWaitL1Done = 8 /* intermediate rows */,
    kErrWaitCombineFlag = 9 /* expert outputs */,
    kErrMetaCapacity = 10, kErrTaskCapacity = 11, kErrWaitFrontend = 12
};
// phase stamp slots (SM 0 unless noted)
enum : int {
    kStampEntry = 0, kStampDispatched = 1, kStampFlagsSeen = 2, kStampScheduled = 3, kStampTasksDone = 4, kStampPrologue = 5 /* SM 0: shared memory, barriers and TMEM are set up */,
    kStampExit = 7, kStampLastExit = 8 /* max over SMs */,
    kStampFrontend = 9, kStampLastTasksDone = 10 /* max over SMs */, kStampLastScheduled = 11 /* max over SMs */,
    kStampLastWeight = 14 /* max over SMs: the last streamed unit has landed */
};

// per-SM phase times (globaltimer ns), slot index inside the SM's 16 records
enum SmPhase : int {
    kSmEntry = 0, kSmPrologue = 1, kSmOwnListed = 2, kSmCountsKnown = 3, kSmScheduled = 4, kSmFirstIssue = 5,
    kSmFirstLanded = 6, kSmFirstStaged = 7, kSmFirstMmaDone = 8, kSmFirstEpilogue = 9, kSmLastL1Epilogue = 10,
    kSmFirstL2Staged = 11, kSmTasksDone = 12, kSmFirstCombined = 13, kSmCombineDone = 14, kSmExit = 15,
    kSmRowsCached = 31 /* a received row has been copied into the row cache (the latest such copy) */
};

struct RowMeta { int32_t src, token, slot; float weight; };

struct KParams {
    int R, rank, e_local, topk, H, I, T, cap;
    int n1_tiles, n2_tiles, k1_units, k2_units;
    int nstage;                          // ring of weight stages, one streamed unit each
    uint32_t unit_bytes;                 // weights + scale planes of one streamed unit
    int x_row_bytes, x_sf_row_bytes, rx_row_bytes, mid_row_bytes, mid_sf_row_bytes;
    float clamp; int has_clamp, fast_math;
    float l1_scale, l2_scale, mid_gs;
    uint8_t* peer[kMaxRanks];
    const uint8_t* w1; const uint8_t* w2;
    __nv_bfloat16* y; int* stats;
    const uint8_t* inp;                  // base of the input views: inp + off_x etc. (the buffer itself, or a mapped host mirror of its input region)
    long long off_ctrl, off_x, off_x_sf, off_topk_idx, off_topk_w, off_rx, off_mid, off_mid_sf, off_comb, off_red, off_cnt;
    int cnt_per_phase;
    long long off_token_tiles, off_mid_tiles, off_arrive;   // operand tile images and their arrival counters (launches with more than 16 rows)
    uint32_t tile_capacity, token_tile_bytes, mid_tile_bytes;
    uint32_t wide_stage_bytes, nstage_wide;   // launches with tile images: stride and depth of the weight ring (it takes over the token staging buffers)
    uint32_t sm_rec, nrec, rec_slot_bytes;    // and a ring of token records of its own (in the token region): offset, slots, bytes of a 32-row record
    long long rx_region;                 // bytes of one (parity, source) region of the receive pool
    uint32_t sm_act, sm_asf, sm_otile, sm_vt;   // dynamic shared memory offsets (stages start at 0)
    uint32_t act_bytes, asf_bytes;
    int ndisp;                           // SMs that share the dispatch to one destination rank
    uint32_t sm_xbuf; int nab;           // widened-unit buffers (FP8 variant); number of 16-row token staging buffers (1 or 2)
    uint32_t stage_region;               // bytes of the token staging area (tiles + scale slots)
    uint32_t sm_rcache, rc_rows, rc_row_bytes;   // row cache: received rows (tokens + scale bytes) fetched before the weight stream starts
    unsigned long long timeout_ns;
    uint32_t knobs;                      // kKnob* bits
    uint32_t pf_w1_max, pf_w2_max;       // experts whose W1 / W2 the scout may prefetch in one launch (L2 capacity)
    FeParams fe; int fe_enabled;         // router frontend run at the head of the same launch (optional)
};

struct Ctl {
    uint64_t full[kMaxStages], empty[kMaxStages];
    uint64_t rfull[kMaxRecSlots], rempty[kMaxRecSlots];   // launches with tile images: ring of token records (record loader -> MMA issuer)
    uint64_t acts_full[2], acts_empty[2], tmem_full[2], tmem_empty[2];
    uint64_t xfull[2], xempty[2];        // FP8-activation variant: widened weight units
    uint64_t meta_full[4], meta_empty[4];   // launches with tile images: the row records of a task's tile (loader -> epilogue)
    uint64_t tile_full;                  // decode mode: the shared token tile is complete (one arrival per filling warp)
    uint32_t tmem_base, epoch, abort_flag, ntasks;
    uint32_t rx_count[kMaxRanks], rx_prefix[kMaxRanks + 1];
    uint32_t exp_count[kMaxLocalExperts], mid_base[kMaxLocalExperts];
    uint32_t nt1, nt2, dcount, own_cnt;
    uint32_t comb_next, issued, decode, bulk;   // next combine item of this SM; weight units the loader has issued; decode mode and tile-image mode (see below)
    // rows of a token tile in this launch (16, or 32 when tile images are in use and an expert has more than 16 rows);
    // queue of finished intermediate tiles, epilogue -> releasing warp
    uint32_t tw, rel_head, rel_tail, rissued;   // (rissued: token records and tile headers the record loader has issued, for the aborted exit)
    uint32_t rel_q[kRelQueue];
    long long rel_t[kRelQueue];          // (wait profile: when the entry was queued)
    uint32_t n1_tasks, padn[3];          // L1 tasks at the head of this SM's list
    uint32_t epi_nv[2], epi_dcol[2];     // per accumulator: valid rows of the task and (decode mode) the first accumulator column of its expert
    // token staging geometry of this launch: with room for one 16-row buffer only, launches whose experts all have at
    // most 8 rows split it into two 8-row buffers (the MMA then reads rows 8..15 from rows 0..7: stride 0 between the
    // 8-row groups; those accumulator columns are never used)
    uint32_t nab, act_stride, atom_stride, sbo;
    uint32_t tasks[kMaxTasks];           // type << 28 | expert << 20 | token tile << 8 | weight tile
    uint32_t tasks2[kMaxTasks];          // first unit | end unit << 8 | parts of the tile << 16 | first contributing SM << 24
    uint32_t tasks3[kMaxTasks];          // tile index inside its phase (counter slot)
    uint32_t red_old;
    RowMeta row_meta[4][kTileTokens];
    RowMeta epi_meta[2][kTileTokens];
    alignas(16) RowMeta meta_ring[4][kWideTokens];
    uint32_t nvalid[4];
    uint32_t rowref[2][kTileTokens];
    uint32_t rowidx[2][kTileTokens];
    uint32_t rcslot[2][kTileTokens];     // row-cache slot of each row of the task being staged (0xFFFFFFFF: not cached)
    float amax_x[4][kTileTokens];
    uint32_t dry_count[kMaxLocalExperts];   // dummy per-expert counts of the schedule's warm-up call
    uint32_t sfb[4][kTileTokens];        // L1 epilogue: one scale byte per (warp, token), gathered into one flagged word
    uint32_t mtl[kMaxMTiles];            // (expert << 16 | token tile) of every 16-token tile, expert-major
    RowMeta rx_meta[kMetaSmemRows];
    RowMeta own_meta[kOwnCap];           // records of this rank's own routed rows, listed by the scout from topk_idx
    uint8_t own_e[kOwnCap];
    alignas(16) uint8_t meta_e[kMetaCap];
};

__device__ __forceinline__ uint32_t task_pack(uint32_t type, uint32_t e, uint32_t mt, uint32_t j) {
    return (type << 28) | (e << 20) | (mt << 8) | j;
}

struct Ctx {
    const KParams& p;
    Ctl& c;
    uint8_t* buf;         // this rank's buffer
    uint8_t* smem;        // dynamic shared memory (1024 B aligned)
    uint64_t deadline;
    uint32_t par;         // launch parity: which half of the receive pool this launch uses (set once the launch number is known)
    bool own_direct;      // rows of this rank's own tokens are read from the caller's input views, not from the receive pool
    __device__ __forceinline__ bool aborted() const { return *reinterpret_cast<volatile uint32_t*>(&c.abort_flag) != 0u; }
    __device__ __noinline__ void fail(uint32_t code, uint32_t detail = 0) const {      // cold: keep it out of the callers' code
        uint32_t* st = reinterpret_cast<uint32_t*>(buf + p.off_ctrl + kCtrlStatus);
        atomicCAS(st, 0u, code | (blockIdx.x << 8) | (detail << 16));
        *reinterpret_cast<volatile uint32_t*>(&c.abort_flag) = 1u;
    }
    __device__ __forceinline__ bool expired() const { return globaltimer_ns() > deadline; }
    // the first probe is inline (a barrier that is already complete costs a few cycles); the polling loop with its
    // abort and deadline checks is one out-of-line copy
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t code) const {
        if (mbar_try_wait(bar, parity)) return true;
        return wait_slow(bar, parity, code);
    }
    __device__ __noinline__ bool wait_slow(uint64_t* bar, uint32_t parity, uint32_t code) const {
        uint32_t it = 0;
        while (!mbar_try_wait(bar, parity)) {
            if ((++it & 0xFFu) == 0u) {
                if (aborted()) return false;
                if (expired()) { fail(code); return false; }
            }
        }
        return true;
    }
    // every lane waits; the warp agrees on the outcome
    __device__ __forceinline__ void wait_total(int slot, long long cycles) const {
        if ((p.knobs & kKnobWaitProfile) != 0u)
            reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmPhase)[blockIdx.x * kSmPhaseSlots + slot] = static_cast<unsigned long long>(cycles);
    }
    __device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, uint32_t code) const {
        return __all_sync(0xffffffffu, wait(bar, parity, code));
    }
    __device__ __forceinline__ void stamp(int slot) const {
        reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlStamps)[slot] = globaltimer_ns();
    }
    __device__ __forceinline__ void sm_phase(int slot) const {
        reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmPhase)[blockIdx.x * kSmPhaseSlots + slot] = globaltimer_ns();
    }
    __device__ __forceinline__ void stamp_max(int slot, unsigned long long t) const {
        atomicMax(reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlStamps) + slot, t);
    }
    // per-SM time of the first weight request of this launch (the scout's first prefetch or the loader's first copy)
    __device__ __forceinline__ void note_first_weight_request() const {
        atomicMin(reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmWFirst) + blockIdx.x, globaltimer_ns());
    }
    // received row i of source rank `src_rank` (flagged words: payload byte b sits at 2 * (b & ~3) + (b & 3))
    __device__ __forceinline__ uint8_t* rx_row(uint32_t src_rank, uint32_t i) const {
        return buf + p.off_rx + static_cast<size_t>(par * p.R + src_rank) * p.rx_region + 32u + static_cast<size_t>(i) * 2u * p.rx_row_bytes;
    }
    // Token rows ahead of the weight stream. The first `rc_rows` received rows (receive order) are fetched into shared
    // memory while the schedule is being built, before the bulk copies of the weight stream make every small load wait
    // behind megabytes. Two uses of the same region: with at most 16 received rows in the launch ("decode mode") they
    // are written straight into ONE swizzled token tile, rows grouped by expert, that every L1 task of the launch
    // multiplies with (a 16-token MMA costs the same whatever rows are meaningful; the task's epilogue reads its
    // expert's accumulator columns); otherwise the region is a plain row cache (slot = receive index) that the stager
    // copies from instead of going to global memory.
    __device__ __forceinline__ uint8_t* tok_region() const { return smem + p.sm_rcache; }
    __device__ __forceinline__ uint8_t* tile_asf() const { return smem + p.sm_rcache + p.act_bytes; }
    // one 16 B payload chunk of flagged words at `src` (32 B): polls until both halves carry this launch's flag
    __device__ __forceinline__ bool ll_read(const uint8_t* src, uint32_t flag, uint4& out, uint32_t code, uint32_t detail) const {
        uint32_t spins = 0;
        for (;;) {
            const uint4 a = ld_volatile_v4(src), b = ld_volatile_v4(src + 16);
            if (ll_valid(a, b, flag)) { out = ll_data(a, b); return true; }
            if ((++spins & 0x3Fu) == 0u) {
                if (aborted()) return false;
                if (expired()) { fail(code, detail); return false; }
            }
        }
    }
};

// position of 16 B chunk `c` of row `r` inside a 128 B-swizzled [rows x 128 B] tile
__device__ __forceinline__ uint32_t sw128_off(uint32_t r, uint32_t c) {
    return (r >> 3) * 1024u + (r & 7u) * 128u + ((c ^ (r & 7u)) << 4);
}
// E2M1 code -> value: the three magnitude bits become the low exponent bit pair and top mantissa bit of an fp16 (x 2^14)
__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const uint32_t h = ((code & 7u) << 9) | ((code & 8u) << 12);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h))) * 16384.0f;
}
template <int kVec>
__device__ __forceinline__ float sf_value(uint32_t byte) {
    if constexpr (kVec == 32) return __uint_as_float((byte & 0xFFu) << 23);
    else return e4m3_to_float(byte);
}

// ============================================================================================= weight loader
__device__ void role_loader(const Ctx& cx) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    uint32_t it = 0, s = 0, ph = 0;                              // units issued; ring stage and its phase bit
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const uint32_t t = c.tasks[ti];
        const uint32_t type = t >> 28, e = (t >> 20) & 0xFF, j = t & 0xFF;
        const int ntiles = type ? p.n2_tiles : p.n1_tiles, kunits = type ? p.k2_units : p.k1_units;
        const uint8_t* src = (type ? p.w2 : p.w1) + (static_cast<size_t>(e) * ntiles + j) * kunits * p.unit_bytes;
        const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
        #pragma unroll 1
        for (int u = ub; u < ue; ++u, ++it) {
            if (!cx.warp_wait(&c.empty[s], ph ^ 1u, kErrWaitEmpty)) return;
            if (elect_one()) {
                mbar_arrive_expect_tx(&c.full[s], p.unit_bytes);
                bulk_g2s(cx.smem + static_cast<size_t>(s) * p.unit_bytes, src + static_cast<size_t>(u) * p.unit_bytes, p.unit_bytes, &c.full[s]);
                c.issued = it + 1u;
                if (it == 0u) { cx.note_first_weight_request(); cx.sm_phase(kSmFirstIssue); }
            }
            __syncwarp();
            if (++s == static_cast<uint32_t>(p.nstage)) { s = 0; ph ^= 1u; }
        }
    }
}

// ============================================================================================= MMA issuer
template <int kVec, bool kA8>
__device__ void role_mma(const Ctx& cx, uint32_t lane) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    constexpr uint32_t kPlanes = kUnitK / (4 * kVec);           // scale words per row per unit
    constexpr uint32_t kIdesc = kA8 ? idesc_block_scaled(kFmtF8E2M1, kFmtF8E4M3, kTileRows, kTileTokens, 1u)
                                    : idesc_block_scaled(kFmtMxf4E2M1, kFmtMxf4E2M1, kTileRows, kTileTokens, kVec == 32 ? 1u : 0u);
    constexpr uint32_t kStepK = kA8 ? 32u : 64u;                // K elements per MMA instruction
    constexpr uint32_t kStepsPerAtom = kA8 ? 4u : 4u;           // 128 B of operand bytes per swizzle atom either way
    const uint32_t tm = c.tmem_base;
    const uint32_t acc_col = 0, sfa_col = 32, sfb_col = 64;     // accumulators 2 x 16, weight scales 2 x 16, token scales 2 x 16
    uint32_t it = 0, s = 0, ph = 0;                             // units consumed so far; ring stage and its phase bit
    unsigned long long t_landed = 0ull;                         // when the latest unit was found in shared memory
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
        const uint32_t acc = ti & 1u, use = (ti >> 1) & 1u;
        // decode mode: every L1 task multiplies with the launch's shared token tile (written once, before the weight
        // stream started); nothing is staged for it and the staging barriers count the L2 tasks only
        const bool shared_tile = !kA8 && c.decode != 0u && (c.tasks[ti] >> 28) == 0u;
        const uint32_t tis = (!kA8 && c.decode != 0u) ? ti - c.n1_tasks : ti;
        const uint32_t ab = c.nab == 2u ? (tis & 1u) : 0u, use_a = c.nab == 2u ? (tis >> 1) & 1u : (tis & 1u);
        if (shared_tile) { if (!cx.warp_wait(&c.tile_full, 0u, kErrWaitActsFull)) return; }
        else if (!cx.warp_wait(&c.acts_full[ab], use_a, kErrWaitActsFull)) return;
        if (!cx.warp_wait(&c.tmem_empty[acc], use ^ 1u, kErrWaitTmemEmpty)) return;
        tc_fence_after();
        const uint32_t act = shared_tile ? smem_u32(cx.tok_region()) : smem_u32(cx.smem + p.sm_act + ab * c.act_stride);
        const uint32_t asf_base = shared_tile ? smem_u32(cx.tile_asf()) : smem_u32(cx.smem + p.sm_asf + ab * p.asf_bytes);
        const uint32_t atom_stride = shared_tile ? kTileTokens * 128u : c.atom_stride, sbo = shared_tile ? 1024u : c.sbo;
        #pragma unroll 1
        for (int u = ub; u < ue; ++u, ++it) {
            uint64_t* ready = kA8 ? &c.xfull[it & 1u] : &c.full[s];
            if (!cx.warp_wait(ready, kA8 ? (it >> 1) & 1u : ph, kErrWaitFull)) return;
            tc_fence_after();
            t_landed = globaltimer_ns();
            if (lane == 0) {
                if (it == 0u) cx.sm_phase(kSmFirstLanded);
                if (it < 15u) cx.sm_phase(16 + static_cast<int>(it));
            }
            if (elect_one()) {
              {
                const uint32_t wsm = kA8 ? smem_u32(cx.smem + p.sm_xbuf + (it & 1u) * kXbufBytes)
                                         : smem_u32(cx.smem + static_cast<size_t>(s) * p.unit_bytes);
                const uint32_t wsf = wsm + (kA8 ? 2u * kUnitWBytes : static_cast<uint32_t>(kUnitWBytes));
                const uint32_t sfa = tm + sfa_col + (it & 1u) * 16u, sfb = tm + sfb_col + (it & 1u) * 16u;
                const uint32_t asf = asf_base + static_cast<uint32_t>(u) * kPlanes * 256u;
                #pragma unroll
                for (uint32_t pl = 0; pl < kPlanes; ++pl) {
                    // one scale word (4 scale bytes, K span 4 * vec) per row: lane = row % 32, column = row / 32.
                    // Token rows fill lanes 0..15 of a plane; lanes 16..31 receive the next plane's bytes and are never read.
                    utccp_32x128b_warpx4(sfa + pl * 4u, smem_desc(wsf + pl * 512u, 128u, kLayoutNone));
                    utccp_32x128b_warpx4(sfb + pl * 4u, smem_desc(asf + pl * 256u, 128u, kLayoutNone));
                }
                // token tile: [K atoms][16 rows x 128 B]; an atom holds 256 packed E2M1 or 128 E4M3 elements
                const uint32_t bsm = act + static_cast<uint32_t>(u) * (kA8 ? 2u : 1u) * atom_stride;
                #pragma unroll
                for (uint32_t ks = 0; ks < kUnitK / kStepK; ++ks) {
                    const uint32_t pl = (ks * kStepK) / (4u * kVec), sf_id = ((ks * kStepK) % (4u * kVec)) / kVec;
                    const uint32_t atom = ks / kStepsPerAtom, in_atom = (ks % kStepsPerAtom) * 32u;
                    const uint64_t adesc = smem_desc(wsm + (kA8 ? atom * kUnitWBytes : 0u) + in_atom, 1024u, kLayoutSw128);
                    const uint64_t bdesc = smem_desc(bsm + (kA8 ? atom * atom_stride : 0u) + in_atom, sbo, kLayoutSw128);
                    const uint32_t idesc = idesc_with_sf(kIdesc, sf_id, sf_id);
                    const uint32_t accum = (u > ub || ks > 0) ? 1u : 0u;
                    if constexpr (kA8)
                        umma_mxf8f6f4(tm + acc_col + acc * 16u, adesc, bdesc, idesc, sfa + pl * 4u, sfb + pl * 4u, accum);
                    else if constexpr (kVec == 32)
                        umma_mxf4_block32(tm + acc_col + acc * 16u, adesc, bdesc, idesc, sfa + pl * 4u, sfb + pl * 4u, accum);
                    else
                        umma_nvf4_block16(tm + acc_col + acc * 16u, adesc, bdesc, idesc, sfa + pl * 4u, sfb + pl * 4u, accum);
                }
              }
              tc_commit(kA8 ? &c.xempty[it & 1u] : &c.empty[s]);
            }
            __syncwarp();
            if (++s == static_cast<uint32_t>(p.nstage)) { s = 0; ph ^= 1u; }
        }
        if (elect_one()) {
            tc_commit(&c.tmem_full[acc]);
            if (!shared_tile) tc_commit(&c.acts_empty[ab]);
        }
        __syncwarp();
    }
    if (lane == 0 && t_landed != 0ull) cx.stamp_max(kStampLastWeight, t_landed);
}

// ============================================================================================= weight widener (FP8 variant)
// kind::mxf8f6f4 reads 4-bit operands from 8-bit-wide shared-memory slots: every 16 E2M1 values (8 bytes) sit in a
// 16-byte slot. HBM keeps the weights packed; four extra warps widen each streamed unit from its packed image
// (128 rows x 128 B, one swizzle atom) into two atoms of 128 rows x 128 B and hand it to the MMA issuer.
__device__ void role_expander(const Ctx& cx, uint32_t xtid) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    // two groups of four warps; group g widens the units of parity g into buffer g, so that one unit's copy overlaps
    // the next unit's barrier round trip
    constexpr uint32_t kGroupThreads = kNumExpThreads / 2;
    const uint32_t lane = xtid & 31u, grp = xtid / kGroupThreads, gt = xtid % kGroupThreads;
    uint8_t* xb = cx.smem + p.sm_xbuf + grp * kXbufBytes;
    uint32_t it = 0, s_next = 0, ph_next = 0;
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
        #pragma unroll 1
        for (int u = ub; u < ue; ++u, ++it) {
            const uint32_t s = s_next, ph = ph_next;
            if (++s_next == static_cast<uint32_t>(p.nstage)) { s_next = 0; ph_next ^= 1u; }
            if ((it & 1u) != grp) continue;
            // every warp waits and signals for itself (the barriers count a group's four warps): no block-level barrier per unit
            if (!cx.warp_wait(&c.full[s], ph, kErrWaitFull)) return;
            if (!cx.warp_wait(&c.xempty[grp], ((it >> 1) & 1u) ^ 1u, kErrWaitEmpty)) return;
            const uint8_t* wsm = cx.smem + static_cast<size_t>(s) * p.unit_bytes;
            // item = (row r, atom a, slot j): the 8 source bytes (16 values) of slot j. Eight consecutive threads fill one
            // widened 128 B row and sixteen read one packed 128 B row: both sides are free of bank conflicts.
            constexpr uint32_t kItems = kTileRows * 16 / kGroupThreads;
            uint2 v[kItems];
            #pragma unroll
            for (uint32_t k = 0; k < kItems; ++k) {
                const uint32_t idx = k * kGroupThreads + gt, j = idx & 7u, at = (idx >> 3) & 1u, r = idx >> 4;
                const uint32_t ch = 4u * at + (j >> 1);
                v[k] = *reinterpret_cast<const uint2*>(wsm + r * 128u + ((ch ^ (r & 7u)) << 4) + (j & 1u) * 8u);
            }
            #pragma unroll
            for (uint32_t k = 0; k < kItems; ++k) {
                const uint32_t idx = k * kGroupThreads + gt, j = idx & 7u, at = (idx >> 3) & 1u, r = idx >> 4;
                *reinterpret_cast<uint4*>(xb + at * kUnitWBytes + r * 128u + ((j ^ (r & 7u)) << 4)) = make_uint4(v[k].x, v[k].y, 0u, 0u);
            }
            if (gt < 64) *reinterpret_cast<uint4*>(xb + 2 * kUnitWBytes + gt * 16u) = *reinterpret_cast<const uint4*>(wsm + kUnitWBytes + gt * 16u);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&c.xfull[grp]); mbar_arrive(&c.empty[s]); }
        }
    }
}

// ============================================================================================= activation stagers
// Rows [16 mt, 16 mt + 16) of local expert e in canonical (source rank, token, slot) order -> c.rowref (flat receive
// index). Executed by one full warp.
__device__ __forceinline__ void find_rows(Ctl& c, uint32_t* rowref, uint32_t total, uint32_t e, uint32_t mt, uint32_t lane) {
    const uint32_t lo = mt * kTileTokens, hi = lo + kTileTokens;
    uint32_t seen = 0;
    #pragma unroll 1
    for (uint32_t base = 0; base < total && seen < hi; base += 32) {
        const uint32_t f = base + lane;
        const bool m = f < total && c.meta_e[f] == e;
        const uint32_t b = __ballot_sync(0xffffffffu, m);
        const uint32_t rank = seen + __popc(b & ((1u << lane) - 1u));
        if (m && rank >= lo && rank < hi) rowref[rank - lo] = f;
        seen += __popc(b);
    }
}

// Two stager warps; warp w stages the tasks with index parity w into staging buffer w, so that two consecutive tasks
// (e.g. a split tile's share and the whole tile that follows) are fetched concurrently.
// `dry`: a rehearsal on two made-up tasks (one of each type, one row, read from row 0 of the own-rank region of the
// receive pool and row 0 of the intermediate pool, whatever they hold; every word accepted, no barrier touched): run
// before the roles start, it leaves this code in the SM's instruction cache, so that the first real task, which sits on
// the launch's critical path, does not pay for fetching it. What it writes into the staging buffer is overwritten later.
__device__ __noinline__ void role_stager(const Ctx& cx, uint32_t sw, uint32_t lane, bool dry) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    const uint32_t total = dry ? 0u : c.rx_prefix[p.R];
    uint32_t* rowref = c.rowref[sw];
    uint32_t* rowidx = c.rowidx[sw];
    uint32_t* rcslot = c.rcslot[sw];
    if (!dry && sw >= c.nab) return;
    bool seen_l2 = false;
    const uint32_t ntasks = dry ? 2u : c.ntasks;
    const uint32_t act_stride = dry ? 0u : c.act_stride, atom_stride = dry ? kTileTokens * 128u : c.atom_stride;
    // In decode mode the L1 tasks use neither the staging buffers nor their barriers (they multiply with the launch's
    // shared token tile and their epilogue lists the rows itself): buffer and phase of a task follow its index among
    // the tasks that do stage, i.e. the L2 tasks.
    const uint32_t skip = (!dry && c.decode != 0u) ? c.n1_tasks : 0u;
    #pragma unroll 1
    for (uint32_t ti = dry ? 0u : skip; ti < ntasks; ++ti) {
        const uint32_t tis = ti - skip;                               // index among the staging tasks
        if (!dry && (c.nab == 2u ? (tis & 1u) : 0u) != sw) continue;   // stager w fills buffer w (one buffer: stager 0 takes every task)
        const uint32_t t = dry ? task_pack(ti, 0u, 0u, 0u) : c.tasks[ti];
        const uint32_t type = t >> 28, e = (t >> 20) & 0xFF, mt = (t >> 8) & 0xFFF;
        const uint32_t ab = (!dry && c.nab == 2u) ? (tis & 1u) : 0u, use = c.nab == 2u ? (tis >> 1) & 1u : (tis & 1u), ring = ti & 3u;
        if (!dry && !cx.warp_wait(&c.acts_empty[ab], use ^ 1u, kErrWaitActsEmpty)) return;
        find_rows(c, rowref, total, e, mt, lane);
        const uint32_t left = c.exp_count[e] - mt * kTileTokens;
        const uint32_t nv = dry ? 1u : (left < kTileTokens ? left : kTileTokens);
        if (lane == 0 && !dry) c.nvalid[ring] = nv;
        __syncwarp();
        if (lane < nv) {
            const uint32_t f = dry ? 0u : rowref[lane];
            uint32_t r = 0;
            while (r + 1 < static_cast<uint32_t>(p.R) && f >= c.rx_prefix[r + 1] && !dry) ++r;
            if (dry) r = static_cast<uint32_t>(p.rank);
            const uint32_t i = dry ? 0u : f - c.rx_prefix[r];
            RowMeta m;
            if (f < kMetaSmemRows) m = c.rx_meta[f];
            else {
                uint4 q = make_uint4(0u, 0u, 0u, 0u);
                cx.ll_read(cx.rx_row(r, i) + 2u * (p.rx_row_bytes - 16), c.epoch + 1u, q, kErrWaitDispatchFlag, r);
                m = RowMeta{0, static_cast<int32_t>(q.y), static_cast<int32_t>(q.z), __uint_as_float(q.w)};
            }
            m.src = static_cast<int32_t>(r);
            if (!dry) c.row_meta[ring][lane] = m;
            rowidx[lane] = (r << 24) | i;
            rcslot[lane] = (dry || f >= p.rc_rows) ? 0xFFFFFFFFu : f;
        }
        __syncwarp();
        uint8_t* act = cx.smem + p.sm_act + ab * act_stride;
        uint8_t* asf = cx.smem + p.sm_asf + ab * p.asf_bytes;
        // Both kinds of rows are flagged words that may still be on their way (received tokens for L1, the L1 epilogues'
        // output of other SMs for L2): a chunk is re-read until its flags match. Received rows carry their scale bytes
        // behind the tokens; intermediate rows keep theirs as one flagged word per (row, L1 tile).
        const uint32_t nchunk = (type ? p.mid_row_bytes : p.x_row_bytes) / 16;             // 16 B chunks of one token row
        const uint32_t per_row = nchunk + (type ? 0u : p.x_sf_row_bytes / 16);
        const uint32_t midrow0 = dry ? 0u : c.mid_base[e] + mt * kTileTokens;
        const uint32_t flag = c.epoch + 1u, wait_code = type ? kErrWaitL1Done : kErrWaitDispatchFlag;
        bool bad = false;
        // one 16 B payload chunk of row n: token bytes into the swizzled tile, scale bytes into their slots
        auto put = [&](uint32_t n, uint32_t ci, const uint4& v) {
            if (ci < nchunk) {
                *reinterpret_cast<uint4*>(act + (ci >> 3) * atom_stride + sw128_off(n, ci & 7u)) = v;
            } else {
                // four scale words: one 16 B slot per (scale word, token), word g of the row at slot g
                uint8_t* dst = asf + (ci - nchunk) * 4u * 256u + n * 16u;
                *reinterpret_cast<uint32_t*>(dst) = v.x;
                *reinterpret_cast<uint32_t*>(dst + 256u) = v.y;
                *reinterpret_cast<uint32_t*>(dst + 512u) = v.z;
                *reinterpret_cast<uint32_t*>(dst + 768u) = v.w;
            }
        };
        #pragma unroll 1
        for (uint32_t n = 0; n < nv; ++n) {
            if (type == 0u && !dry && p.rc_rows != 0u) {
                // a row that was fetched into the row cache before the weight stream started: shared memory to shared memory
                const uint32_t slot = rcslot[n];
                if (slot != 0xFFFFFFFFu) {
                    const uint8_t* src = cx.smem + p.sm_rcache + slot * p.rc_row_bytes;
                    #pragma unroll 1
                    for (uint32_t ci = lane; ci < per_row; ci += 32) put(n, ci, *reinterpret_cast<const uint4*>(src + ci * 16u));
                    continue;
                }
            }
            if (type == 0u && !dry && cx.own_direct && (rowidx[n] >> 24) == static_cast<uint32_t>(p.rank)) {
                // a row of this rank's own token (not in the row cache): the token where the caller put it, plain loads
                const uint32_t tok = static_cast<uint32_t>(c.row_meta[ring][n].token);
                const uint8_t* xs = p.inp + p.off_x + static_cast<size_t>(tok) * p.x_row_bytes;
                const uint8_t* sf = p.inp + p.off_x_sf + static_cast<size_t>(tok) * p.x_sf_row_bytes;
                #pragma unroll 1
                for (uint32_t ci = lane; ci < per_row; ci += 32)
                    put(n, ci, ld_cg_v4(ci < nchunk ? xs + ci * 16u : sf + (ci - nchunk) * 16u));
                continue;
            }
            const uint8_t* row_src = type ? cx.buf + p.off_mid + static_cast<size_t>(midrow0 + n) * 2u * p.mid_row_bytes
                                          : cx.rx_row(rowidx[n] >> 24, rowidx[n] & 0xFFFFFFu);
            // four chunks per lane are in flight before the first store: one memory round trip per 128 chunks of a row
            #pragma unroll 1
            for (uint32_t base = lane; base < per_row; base += 4 * 32) {
                uint4 v[4];
                uint32_t spins = 0;
                bool ok;
                do {
                    ok = true;
                    #pragma unroll
                    for (uint32_t u = 0; u < 4; ++u) {
                        const uint32_t ci = base + u * 32;
                        if (ci < per_row) {
                            const uint4 a = ld_volatile_v4(row_src + ci * 32u), b = ld_volatile_v4(row_src + ci * 32u + 16u);
                            ok = ok && (ll_valid(a, b, flag) || dry);
                            v[u] = ll_data(a, b);
                        }
                    }
                    if (!ok && (++spins & 0x3Fu) == 0u) {
                        if (cx.aborted()) bad = true;
                        else if (cx.expired()) { cx.fail(wait_code, type ? e : rowidx[n] >> 24); bad = true; }
                    }
                } while (!ok && !bad);
                #pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t ci = base + u * 32;
                    if (ci < per_row) put(n, ci, v[u]);
                }
            }
            if (type) {
                // scale bytes of the intermediate row: L1 tile w wrote {2 bytes (one per 32 columns) or 4 bytes (one per 16), flag}
                const uint8_t* sf_src = cx.buf + p.off_mid_sf + static_cast<size_t>(midrow0 + n) * p.n1_tiles * 8u;
                #pragma unroll 1
                for (uint32_t w = lane; w < static_cast<uint32_t>(p.n1_tiles); w += 32) {
                    uint32_t spins = 0;
                    uint2 q;
                    for (;;) {
                        q = ld_volatile_v2(sf_src + w * 8u);
                        if (q.y == flag || bad || dry) break;
                        if ((++spins & 0x3Fu) == 0u) {
                            if (cx.aborted()) bad = true;
                            else if (cx.expired()) { cx.fail(kErrWaitL1Done, e); bad = true; }
                        }
                    }
                    if (p.x_sf_row_bytes * 16 == p.H)           // one scale byte per 16 elements: four bytes per tile, one scale word
                        *reinterpret_cast<uint32_t*>(asf + w * 256u + n * 16u) = q.x;
                    else                                          // per 32 elements: two bytes per tile, half a scale word
                        *reinterpret_cast<uint16_t*>(asf + (w >> 1) * 256u + n * 16u + (w & 1u) * 2u) = static_cast<uint16_t>(q.x);
                }
            }
        }
        if (__any_sync(0xffffffffu, bad)) return;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && !dry) {
            mbar_arrive(&c.acts_full[ab]);
            if (tis == 0u) cx.sm_phase(kSmFirstStaged);
            if (type != 0u && !seen_l2) { seen_l2 = true; cx.sm_phase(kSmFirstL2Staged); }
        }
    }
}

// ============================================================================================= epilogue
// CUDA-core evaluation of one streamed unit for one weight row (the on-device cross-check of the tensor-core path):
// v[n] += sum_k w[row][k] a[n][k] with both operands' block scales applied.
template <int kVec>
__device__ __forceinline__ void check_accumulate(const Ctx& cx, const uint8_t* wsm, const uint8_t* act, const uint8_t* asf,
                                                 uint32_t u, uint32_t row, uint32_t nv, float (&v)[kTileTokens]) {
    constexpr uint32_t kPlanes = kUnitK / (4 * kVec);
    constexpr uint32_t kBlockBytes = kVec / 2;
    const uint8_t* wrow = wsm + (row >> 3) * 1024u + (row & 7u) * 128u;
    const uint32_t* wsf = reinterpret_cast<const uint32_t*>(wsm + kUnitWBytes);
    #pragma unroll
    for (uint32_t pl = 0; pl < kPlanes; ++pl) {
        const uint32_t wword = wsf[pl * 128u + (row & 31u) * 4u + (row >> 5)];
        const uint32_t g = u * kPlanes + pl;
        #pragma unroll
        for (uint32_t sb = 0; sb < 4; ++sb) {
            const float sw = sf_value<kVec>((wword >> (8 * sb)) & 0xFFu);
            const uint32_t byte0 = (pl * 4u + sb) * kBlockBytes;            // byte offset inside the 128 B row
            const uint32_t ci = byte0 >> 4, in = byte0 & 15u;
            uint32_t wq[kBlockBytes / 4];
            #pragma unroll
            for (uint32_t w4 = 0; w4 < kBlockBytes / 4; ++w4)
                wq[w4] = *reinterpret_cast<const uint32_t*>(wrow + ((ci ^ (row & 7u)) << 4) + in + w4 * 4u);
            #pragma unroll
            for (uint32_t n = 0; n < kTileTokens; ++n) {
                if (n < nv) {
                    const uint8_t* arow = act + u * (kTileTokens * 128u) + (n >> 3) * 1024u + (n & 7u) * 128u + ((ci ^ (n & 7u)) << 4) + in;
                    const uint32_t aword = *reinterpret_cast<const uint32_t*>(asf + g * 256u + n * 16u);
                    const float sa = sf_value<kVec>((aword >> (8 * sb)) & 0xFFu);
                    float dot = 0.f;
                    #pragma unroll
                    for (uint32_t w4 = 0; w4 < kBlockBytes / 4; ++w4) {
                        const uint32_t aq = *reinterpret_cast<const uint32_t*>(arow + w4 * 4u);
                        #pragma unroll
                        for (uint32_t k = 0; k < 8; ++k)
                            dot += e2m1_value((wq[w4] >> (4 * k)) & 0xFu) * e2m1_value((aq >> (4 * k)) & 0xFu);
                    }
                    v[n] += dot * sw * sa;
                }
            }
        }
    }
}

template <int kVec, bool kUmma, bool kA8>
__device__ void role_epilogue(const Ctx& cx, uint32_t etid) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    const uint32_t ew = etid >> 5, lane = etid & 31u, row = etid;
    uint8_t* otile = cx.smem + p.sm_otile;
    float* vt = reinterpret_cast<float*>(cx.smem + p.sm_vt) + row;      // this thread's accumulators: vt[n * 128], token n
    uint32_t it = 0;
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const uint32_t t = c.tasks[ti];
        const uint32_t type = t >> 28, e = (t >> 20) & 0xFF, mt = (t >> 8) & 0xFFF, j = t & 0xFF;
        const uint32_t acc = ti & 1u, use = (ti >> 1) & 1u, ring = ti & 3u, ab = c.nab == 2u ? acc : 0u;
        float* vtt = vt;                                           // this task's accumulators: vtt[n * 128], token n of the task
        // ---- accumulators of the valid tokens -> shared memory (the loops below run over the valid tokens only)
        bool ok;
        uint32_t nv = 0;
        if constexpr (kUmma) {
            ok = cx.warp_wait(&c.tmem_full[acc], use, kErrWaitTmemFull);
            // decode mode, L1 task: nobody staged anything for this task (its tokens sit in the launch's shared tile). The
            // first epilogue warp lists the expert's rows itself, in receive order: their records, how many there are, and
            // how many rows of experts with a smaller index precede them in the tile (= the expert's first column).
            const bool shared_tile = !kA8 && type == 0u && c.decode != 0u;
            if (ok) {
                tc_fence_after();
                if (ti == 0u && etid == 0u) cx.sm_phase(kSmFirstMmaDone);
                if (shared_tile) {
                    if (ew == 0u) {
                        const uint32_t total = c.rx_prefix[p.R];
                        const uint32_t my_e = lane < total ? c.meta_e[lane] : 0xFFu;
                        const uint32_t same = __ballot_sync(0xffffffffu, my_e == e), below = __ballot_sync(0xffffffffu, my_e < e);
                        if (my_e == e) {
                            uint32_t r = 0;
                            while (r + 1 < static_cast<uint32_t>(p.R) && lane >= c.rx_prefix[r + 1]) ++r;
                            RowMeta m = c.rx_meta[lane];
                            m.src = static_cast<int32_t>(r);
                            c.epi_meta[acc][__popc(same & ((1u << lane) - 1u))] = m;
                        }
                        if (lane == 0) { c.epi_nv[acc] = __popc(same); c.epi_dcol[acc] = __popc(below); }
                    }
                } else {
                    if (etid < kTileTokens) c.epi_meta[acc][etid] = c.row_meta[ring][etid];
                    if (etid == 0u) { c.epi_nv[acc] = c.nvalid[ring]; c.epi_dcol[acc] = 0u; }
                }
                uint32_t raw[kTileTokens];
                tmem_ld_32x32b_x16(c.tmem_base + ((ew * 32u) << 16) + acc * 16u, raw);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(&c.tmem_empty[acc]);
                // all sixteen columns go to shared memory (in decode mode they are every received row of the launch; this
                // task's expert owns nv of them from its first column on)
                #pragma unroll
                for (int n = 0; n < kTileTokens; ++n) vt[n * kTileRows] = __uint_as_float(raw[n]);
            }
        } else {
            ok = cx.warp_wait(&c.acts_full[ab], use, kErrWaitActsFull);
            if (ok) {
                if (etid < kTileTokens) c.epi_meta[acc][etid] = c.row_meta[ring][etid];
                nv = c.nvalid[ring];
                if (etid == 0u) { c.epi_nv[acc] = nv; c.epi_dcol[acc] = 0u; }
                float v[kTileTokens];
                #pragma unroll
                for (int n = 0; n < kTileTokens; ++n) v[n] = 0.f;
                const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
                const uint8_t* act = cx.smem + p.sm_act + ab * c.act_stride;
                const uint8_t* asf = cx.smem + p.sm_asf + ab * p.asf_bytes;
                #pragma unroll 1
                for (int u = ub; u < ue && ok; ++u, ++it) {
                    const uint32_t s = it % p.nstage, ph = (it / p.nstage) & 1u;      // cross-check engine: not a fast path
                    ok = cx.warp_wait(&c.full[s], ph, kErrWaitFull);
                    if (ok) {
                        check_accumulate<kVec>(cx, cx.smem + static_cast<size_t>(s) * p.unit_bytes, act, asf, u, row, nv, v);
                        mbar_arrive(&c.empty[s]);
                    }
                }
                if (ok) mbar_arrive(&c.acts_empty[ab]);
                #pragma unroll
                for (int n = 0; n < kTileTokens; ++n) if (n < static_cast<int>(nv)) vt[n * kTileRows] = v[n];
            }
        }
        if (bar_red_or(kBarEpi, kNumEpiThreads, !ok)) return;        // also publishes epi_meta, epi_nv, epi_dcol
        nv = c.epi_nv[acc];
        vtt = vt + c.epi_dcol[acc] * kTileRows;
        const RowMeta* meta = c.epi_meta[acc];
        const uint32_t midrow0 = c.mid_base[e] + mt * kTileTokens;
        const uint32_t np = (c.tasks2[ti] >> 16) & 0xFFu;
        if (np > 1u) {
            // this SM covered only part of the tile's K range: park the partial sums, count in, and let the last
            // contributor add the parts in SM order (a fixed order: the result does not depend on who arrives last)
            const uint32_t tile = c.tasks3[ti], cfirst = c.tasks2[ti] >> 24;
            float* red = reinterpret_cast<float*>(cx.buf + p.off_red);
            float* mine = red + ((static_cast<size_t>(blockIdx.x) * 2u + type) * 2u) * (kTileTokens * kTileRows) + row;
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) mine[n * kTileRows] = vtt[n * kTileRows];
            bar_sync(kBarEpi, kNumEpiThreads);
            if (etid == 0) {
                uint32_t* cnt = reinterpret_cast<uint32_t*>(cx.buf + p.off_cnt) + type * p.cnt_per_phase + tile;
                const uint32_t old = atom_acq_rel_gpu_add(cnt, 1u);
                if (old == np - 1u) *cnt = 0u;
                c.red_old = old;
            }
            bar_sync(kBarEpi, kNumEpiThreads);
            if (c.red_old != np - 1u) continue;
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) {
                float sum = 0.f;
                #pragma unroll 1
                for (uint32_t pc0 = 0; pc0 < np; pc0 += 4) {          // four parts' loads in flight together, added in SM order
                    float part_v[4];
                    #pragma unroll
                    for (uint32_t d = 0; d < 4; ++d) {
                        const uint32_t g = cfirst + pc0 + d;
                        part_v[d] = 0.f;
                        if (pc0 + d < np) {
                            const float* part = red + ((static_cast<size_t>(g) * 2u + type) * 2u) * (kTileTokens * kTileRows);
                            part_v[d] = __uint_as_float(ld_cg_u32(part + n * kTileRows + row));
                        }
                    }
                    #pragma unroll
                    for (uint32_t d = 0; d < 4; ++d) if (pc0 + d < np) sum += part_v[d];
                }
                vtt[n * kTileRows] = sum;
            }
        }

        if (type == 0u) {
            // ---- L1: rows come in groups of 16 = 8 gate rows then the 8 matching up rows
            const bool is_up = (lane & 8u) != 0u;
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) {
                const float mine = bf16_round(vtt[n * kTileRows] * p.l1_scale);
                const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
                float gate = is_up ? other : mine, up = is_up ? mine : other;
                if (p.has_clamp) { gate = fminf(gate, p.clamp); up = fminf(fmaxf(up, -p.clamp), p.clamp); }
                const float sig = p.fast_math ? __frcp_rn(1.0f + __expf(-gate)) : 1.0f / (1.0f + expf(-gate));
                float av = gate * sig * up * meta[n].weight;
                if constexpr (kVec == 16) av = __fdiv_rn(av, p.mid_gs);
                vtt[n * kTileRows] = av;
                float a = fabsf(av);
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
                if (lane == 0) c.amax_x[ew][n] = a;
            }
            if constexpr (kVec == 32) bar_sync(kBarEpi, kNumEpiThreads);     // a 32-column scale block spans two warps
            else __syncwarp();
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) {
                float amax = c.amax_x[ew][n];
                if constexpr (kVec == 32) amax = fmaxf(amax, c.amax_x[ew ^ 1u][n]);
                amax = fmaxf(amax, 1e-30f);
                const float av = vtt[n * kTileRows];
                uint32_t sf_byte; float scaled;
                if constexpr (kA8) {
                    sf_byte = ceil_pow2_exp(__fdiv_rn(amax, 448.0f));
                    scaled = __fdiv_rn(av, __uint_as_float(sf_byte << 23));
                } else if constexpr (kVec == 32) {
                    sf_byte = ceil_pow2_exp(__fdiv_rn(amax, 6.0f));
                    scaled = __fdiv_rn(av, __uint_as_float(sf_byte << 23));
                } else {
                    sf_byte = cvt_e4m3x2(__fdiv_rn(amax, 6.0f), 0.f) & 0xFFu;
                    const float sf = e4m3_to_float(sf_byte);
                    scaled = sf > 0.f ? __fdiv_rn(av, sf) : (av == 0.f ? 0.f : copysignf(6.0f, av));
                }
                const float nb = __shfl_down_sync(0xffffffffu, scaled, 1);
                if (!is_up && (lane & 1u) == 0u) {
                    if constexpr (kA8)
                        *reinterpret_cast<uint16_t*>(otile + n * 64u + ew * 16u + (lane >> 4) * 8u + (lane & 7u)) = static_cast<uint16_t>(cvt_e4m3x2(scaled, nb));
                    else
                        otile[n * 32 + ew * 8u + (lane >> 4) * 4u + ((lane & 7u) >> 1)] = static_cast<uint8_t>(cvt_e2m1x2(scaled, nb));
                }
                if (lane == 0) c.sfb[ew][n] = sf_byte;
            }
            bar_sync(kBarEpi, kNumEpiThreads);
            {
                // The intermediate rows go out as flagged words (the L2 stagers of all SMs poll the data itself: no
                // counter, no release fence): 16 B chunks of the token's 64 output columns, and one word with this
                // tile's scale bytes.
                constexpr uint32_t kChunks = kA8 ? 4u : 2u;
                const uint32_t flag = c.epoch + 1u;
                if (etid < nv * kChunks) {
                    const uint32_t n = etid / kChunks, q16 = etid % kChunks;
                    const uint4 val = *reinterpret_cast<const uint4*>(otile + (n * kChunks + q16) * 16u);
                    st_ll_16B(cx.buf + p.off_mid + static_cast<size_t>(midrow0 + n) * 2u * p.mid_row_bytes + (j * kChunks + q16) * 32u, val, flag);
                } else if (etid >= 64u && etid - 64u < nv) {
                    const uint32_t n = etid - 64u;
                    const uint32_t word = kVec == 16 ? (c.sfb[0][n] | (c.sfb[1][n] << 8) | (c.sfb[2][n] << 16) | (c.sfb[3][n] << 24))
                                                     : (c.sfb[0][n] | (c.sfb[2][n] << 8));
                    st_volatile_v2(cx.buf + p.off_mid_sf + (static_cast<size_t>(midrow0 + n) * p.n1_tiles + j) * 8u, word, flag);
                }
            }
        } else {
            // ---- L2: bf16 rows back to the token's source rank, as flagged words: the combine there polls the data itself
            __nv_bfloat16* ot = reinterpret_cast<__nv_bfloat16*>(otile);
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) ot[n * kTileRows + row] = __float2bfloat16_rn(vtt[n * kTileRows] * p.l2_scale);
            bar_sync(kBarEpi, kNumEpiThreads);
            // (two lanes per 16 B chunk, one 16 B half of its flagged image each: full 32 B sectors per store instruction)
            #pragma unroll 1
            for (uint32_t idx = etid; idx < nv * 32u; idx += kNumEpiThreads) {
                const uint32_t n = idx >> 5, ch = (idx & 31u) >> 1;
                const uint4 val = *reinterpret_cast<const uint4*>(otile + n * 256u + ch * 16u);
                uint8_t* dst = p.peer[meta[n].src] + p.off_comb +
                    ((static_cast<size_t>(meta[n].token) * p.topk + meta[n].slot) * p.H + j * kTileRows) * 4u + ch * 32u;
                st_ll_half(dst, val, c.epoch + 1u, idx & 1u);
            }
        }
        if (etid == 0u) {
            if (ti == 0u) cx.sm_phase(kSmFirstEpilogue);
            if (type == 0u) cx.sm_phase(kSmLastL1Epilogue);
        }
    }
}

// ============================================================================================= roles with tile images
// Launches with more than 16 received rows. The rows have been sorted into tile images in global memory (token tiles by
// the sorting pass after the dispatch, intermediate tiles by the L1 epilogues): per tile and per streamed K unit one
// record = the unit's 128 B of every token row in the tensor core's swizzled order, then the unit's scale-word slots.
// A record travels beside its weight unit: one warp streams the weight units into the weight ring (which takes over the
// space of the token staging buffers), another the records into a ring of record slots in the token region; the MMA
// issuer waits for both copies of a unit. A task needs no token staging of its own and the token operand costs one bulk
// copy per unit, whatever the weight flood does to small loads. A token tile has `c.tw` rows: 16, or 32 when an expert
// has more than 16 rows (the block-scaled MMA takes the same time for 16 and 32 columns: an expert's weights stream
// once for up to 32 rows).
// The launch parameters the tile-image roles use, handed to them by value (in registers).
struct TileP {
    uint32_t unit_bytes, wide_stage_bytes, nstage_wide, tile_capacity, token_tile_bytes, mid_tile_bytes, sm_vt, knobs, sm_rec, nrec, rec_slot_bytes;
    int n1_tiles, n2_tiles, k1_units, k2_units, topk, H, has_clamp, fast_math, cnt_per_phase;
    float clamp, l1_scale, l2_scale, mid_gs;
    long long off_mid_tiles, off_token_tiles, off_arrive, off_red, off_cnt, off_comb;
    const uint8_t* w1; const uint8_t* w2;
};
__device__ __forceinline__ TileP make_tile_params(const KParams& p) {
    TileP t;
    t.sm_rec = p.sm_rec; t.nrec = p.nrec; t.rec_slot_bytes = p.rec_slot_bytes;
    t.unit_bytes = p.unit_bytes; t.wide_stage_bytes = p.wide_stage_bytes; t.nstage_wide = p.nstage_wide; t.tile_capacity = p.tile_capacity;
    t.token_tile_bytes = p.token_tile_bytes; t.mid_tile_bytes = p.mid_tile_bytes; t.sm_vt = p.sm_vt; t.knobs = p.knobs;
    t.n1_tiles = p.n1_tiles; t.n2_tiles = p.n2_tiles; t.k1_units = p.k1_units; t.k2_units = p.k2_units; t.topk = p.topk; t.H = p.H;
    t.has_clamp = p.has_clamp; t.fast_math = p.fast_math; t.cnt_per_phase = p.cnt_per_phase;
    t.clamp = p.clamp; t.l1_scale = p.l1_scale; t.l2_scale = p.l2_scale; t.mid_gs = p.mid_gs;
    t.off_mid_tiles = p.off_mid_tiles; t.off_token_tiles = p.off_token_tiles; t.off_arrive = p.off_arrive; t.off_red = p.off_red;
    t.off_cnt = p.off_cnt; t.off_comb = p.off_comb; t.w1 = p.w1; t.w2 = p.w2;
    return t;
}
// the roles' own wait (first probe inline, timed only when the wait profile is on) and profile helpers
struct TileCtx {
    const Ctx& cx; bool prof;
    __device__ __forceinline__ long long clk() const { return prof ? clock64() : 0ll; }
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t code, long long& acc) const {
        if (!prof) return cx.warp_wait(bar, parity, code);
        const long long t0 = clock64();
        const bool ok = cx.warp_wait(bar, parity, code);
        acc += clock64() - t0;
        return ok;
    }
    __device__ __forceinline__ void total(int slot, long long cycles) const { if (prof) cx.wait_total(slot, cycles); }
};
__device__ __forceinline__ uint32_t tile_record_bytes(uint32_t tw, uint32_t planes) { return tw * 128u + planes * tw * 16u; }

// Weight units of this SM's tasks into the weight ring of the tile-image launches (the same stream as `role_loader`, more stages).
__device__ void role_loader_tiles(const Ctx& cx, const TileP p) {
    Ctl& c = cx.c;
    uint8_t* const smem = cx.smem;
    const TileCtx tc{cx, (p.knobs & kKnobWaitProfile) != 0u};
    uint32_t it = 0, s = 0, ph = 0;
    long long w_empty = 0;
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const uint32_t t = c.tasks[ti];
        const uint32_t type = t >> 28, e = (t >> 20) & 0xFF, j = t & 0xFF;
        const int ntiles = type ? p.n2_tiles : p.n1_tiles, kunits = type ? p.k2_units : p.k1_units;
        const uint8_t* src = (type ? p.w2 : p.w1) + (static_cast<size_t>(e) * ntiles + j) * kunits * p.unit_bytes;
        const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
        #pragma unroll 1
        for (int u = ub; u < ue; ++u, ++it) {
            if (!tc.wait(&c.empty[s], ph ^ 1u, kErrWaitEmpty, w_empty)) return;
            if (elect_one()) {
                mbar_arrive_expect_tx(&c.full[s], p.unit_bytes);
                bulk_g2s(smem + static_cast<size_t>(s) * p.wide_stage_bytes, src + static_cast<size_t>(u) * p.unit_bytes, p.unit_bytes, &c.full[s]);
                c.issued = it + 1u;
                if (it == 0u) { cx.note_first_weight_request(); cx.sm_phase(kSmFirstIssue); }
            }
            __syncwarp();
            if (++s == p.nstage_wide) { s = 0; ph ^= 1u; }
        }
    }
    if ((threadIdx.x & 31u) == 0u) tc.total(16, w_empty);
}

// The token side of the same stages, by a warp of its own: per task the row records of its tile (for the epilogue), per
// unit the tile's record. This warp waits for tiles that are not complete yet; the weight loader never does, so the
// weights of the following units keep coming while a tile is awaited.
__device__ void role_record_loader(const Ctx& cx, const TileP p, uint32_t planes) {
    Ctl& c = cx.c;
    uint8_t* const smem = cx.smem; uint8_t* const buf = cx.buf; const uint32_t par = cx.par;
    const TileCtx tc{cx, (p.knobs & kKnobWaitProfile) != 0u};
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t tw = c.tw, rec = tile_record_bytes(tw, planes);
    const uint32_t* arrive = reinterpret_cast<const uint32_t*>(buf + p.off_arrive) + par * 2u * p.tile_capacity;
    uint32_t s = 0, ph = 0, nissued = 0;
    long long w_tiles = 0;
    // Whether a task's tile is complete (L1: its received rows, L2: the outputs of all L1 weight tiles, counted into the
    // tile's arrival word) is looked up for 32 tasks at a time, one lane per task: one memory round trip per window.
    uint32_t win_base = 0, win_ready = 0;
    auto refresh = [&](uint32_t base) {
        const uint32_t ti = base + lane;
        bool r = false;
        if (ti < c.ntasks) {
            const uint32_t t = c.tasks[ti], type = t >> 28, e = (t >> 20) & 0xFF, mt = (t >> 8) & 0xFFF;
            const uint32_t tile = udiv_small(c.mid_base[e], tw) + mt, left = c.exp_count[e] - mt * tw;
            const uint32_t need = type ? static_cast<uint32_t>(p.n1_tiles) : (left < tw ? left : tw);
            r = ld_acquire_gpu(arrive + type * p.tile_capacity + tile) >= need;
        }
        win_base = base;
        win_ready = __ballot_sync(0xffffffffu, r);
    };
    refresh(0u);
    fence_proxy_async_all();           // the rows were written through the generic proxy; the bulk copies read them through the async proxy
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const uint32_t t = c.tasks[ti];
        const uint32_t type = t >> 28, e = (t >> 20) & 0xFF, mt = (t >> 8) & 0xFFF;
        const uint32_t tile = udiv_small(c.mid_base[e], tw) + mt;
        const uint8_t* head = buf + p.off_token_tiles + static_cast<size_t>(tile) * p.token_tile_bytes;
        const uint8_t* img = type ? buf + p.off_mid_tiles + static_cast<size_t>(tile) * p.mid_tile_bytes : head + kWideTokens * 16u;
        if (!(ti - win_base < 32u && ((win_ready >> (ti - win_base)) & 1u) != 0u)) {
            const long long t0 = tc.clk();
            uint32_t spins = 0;
            for (;;) {
                refresh(ti);
                if (win_ready & 1u) break;
                if ((++spins & 0xFu) == 0u) {
                    if (cx.aborted()) return;
                    if (cx.expired()) { cx.fail(type ? kErrWaitL1Done : kErrWaitDispatchFlag, e); return; }
                }
            }
            fence_proxy_async_all();
            w_tiles += tc.clk() - t0;
        }
        {
            // the rows' records (source rank, token, slot, top-k weight) of the task's tile, for its epilogue: slot ti mod 4
            const uint32_t ms = ti & 3u;
            if (!cx.warp_wait(&c.meta_empty[ms], ((ti >> 2) & 1u) ^ 1u, kErrWaitEmpty)) return;
            if (elect_one()) {
                mbar_arrive_expect_tx(&c.meta_full[ms], kWideTokens * 16u);
                bulk_g2s(c.meta_ring[ms], head, kWideTokens * 16u, &c.meta_full[ms]);
            }
            __syncwarp();
        }
        const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
        #pragma unroll 1
        for (int u = ub; u < ue; ++u) {
            if (!cx.warp_wait(&c.rempty[s], ph ^ 1u, kErrWaitEmpty)) return;
            if (elect_one()) {
                mbar_arrive_expect_tx(&c.rfull[s], rec);
                bulk_g2s(smem + p.sm_rec + static_cast<size_t>(s) * p.rec_slot_bytes, img + static_cast<size_t>(u) * rec, rec, &c.rfull[s]);
                c.rissued = ++nissued;
            }
            __syncwarp();
            if (++s == p.nrec) { s = 0; ph ^= 1u; }
        }
    }
    if (lane == 0u) tc.total(17, w_tiles);
}

template <int kVec>
__device__ void role_mma_tiles(const Ctx& cx, const TileP p, uint32_t lane) {
    Ctl& c = cx.c;
    uint8_t* const smem = cx.smem;
    const TileCtx tc{cx, (p.knobs & kKnobWaitProfile) != 0u};
    constexpr uint32_t kPlanes = kUnitK / (4 * kVec);
    const uint32_t tw = c.tw;
    const uint32_t idesc0 = idesc_block_scaled(kFmtMxf4E2M1, kFmtMxf4E2M1, kTileRows, tw, kVec == 32 ? 1u : 0u);
    const uint32_t tm = c.tmem_base;
    const uint32_t sfa_col = 64, sfb_col = 96;                  // accumulators 2 x 32 columns, weight scales 2 x 16, token scales 2 x 16
    uint32_t it = 0, s = 0, ph = 0, rs = 0, rph = 0;             // units consumed; weight stage and record slot with their phase bits
    unsigned long long t_landed = 0ull;
    long long w_tmem = 0, w_full = 0, w_tok = 0;
    const long long t_role = tc.clk();
    const unsigned long long ns_role = tc.prof ? globaltimer_ns() : 0ull;
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const int ub = c.tasks2[ti] & 0xFF, ue = (c.tasks2[ti] >> 8) & 0xFF;
        const uint32_t acc = ti & 1u, use = (ti >> 1) & 1u;
        if (!tc.wait(&c.tmem_empty[acc], use ^ 1u, kErrWaitTmemEmpty, w_tmem)) return;
        tc_fence_after();
        #pragma unroll 1
        for (int u = ub; u < ue; ++u, ++it) {
            if (!tc.wait(&c.full[s], ph, kErrWaitFull, w_full)) return;
            if (!tc.wait(&c.rfull[rs], rph, kErrWaitActsFull, w_tok)) return;
            tc_fence_after();
            t_landed = globaltimer_ns();
            if (lane == 0 && it == 0u) cx.sm_phase(kSmFirstLanded);
            if (elect_one()) {
                const uint32_t wsm = smem_u32(smem + static_cast<size_t>(s) * p.wide_stage_bytes);
                const uint32_t wsf = wsm + static_cast<uint32_t>(kUnitWBytes);
                const uint32_t tok = smem_u32(smem + p.sm_rec + static_cast<size_t>(rs) * p.rec_slot_bytes), tsf = tok + tw * 128u;
                const uint32_t sfa = tm + sfa_col + (it & 1u) * 16u, sfb = tm + sfb_col + (it & 1u) * 16u;
                #pragma unroll
                for (uint32_t pl = 0; pl < kPlanes; ++pl) {
                    utccp_32x128b_warpx4(sfa + pl * 4u, smem_desc(wsf + pl * 512u, 128u, kLayoutNone));
                    // (16-row tiles: the copy's upper 16 lanes read the next plane, or the unused tail of the stage)
                    utccp_32x128b_warpx4(sfb + pl * 4u, smem_desc(tsf + pl * tw * 16u, 128u, kLayoutNone));
                }
                #pragma unroll
                for (uint32_t ks = 0; ks < kUnitK / 64u; ++ks) {
                    const uint32_t pl = (ks * 64u) / (4u * kVec), sf_id = ((ks * 64u) % (4u * kVec)) / kVec;
                    const uint64_t adesc = smem_desc(wsm + ks * 32u, 1024u, kLayoutSw128);
                    const uint64_t bdesc = smem_desc(tok + ks * 32u, 1024u, kLayoutSw128);
                    const uint32_t idesc = idesc_with_sf(idesc0, sf_id, sf_id);
                    const uint32_t accum = (u > ub || ks > 0) ? 1u : 0u;
                    if constexpr (kVec == 32)
                        umma_mxf4_block32(tm + acc * kWideTokens, adesc, bdesc, idesc, sfa + pl * 4u, sfb + pl * 4u, accum);
                    else
                        umma_nvf4_block16(tm + acc * kWideTokens, adesc, bdesc, idesc, sfa + pl * 4u, sfb + pl * 4u, accum);
                }
                tc_commit(&c.empty[s]);
                tc_commit(&c.rempty[rs]);
            }
            __syncwarp();
            if (++s == p.nstage_wide) { s = 0; ph ^= 1u; }
            if (++rs == p.nrec) { rs = 0; rph ^= 1u; }
        }
        if (elect_one()) tc_commit(&c.tmem_full[acc]);
        __syncwarp();
    }
    if (lane == 0 && t_landed != 0ull) cx.stamp_max(kStampLastWeight, t_landed);
    if (lane == 0) {
        tc.total(18, w_tmem); tc.total(19, w_full); tc.total(20, tc.clk() - t_role);
        if (tc.prof) tc.total(25, static_cast<long long>(globaltimer_ns() - ns_role)); tc.total(26, w_tok);
    }
}

template <int kVec>
__device__ void role_epilogue_tiles(const Ctx& cx, const TileP p, uint32_t etid) {
    Ctl& c = cx.c;
    uint8_t* const smem = cx.smem; uint8_t* const buf = cx.buf; const uint32_t par = cx.par;
    const TileCtx tc{cx, (p.knobs & kKnobWaitProfile) != 0u};
    constexpr uint32_t kPlanes = kUnitK / (4 * kVec);
    const uint32_t ew = etid >> 5, lane = etid & 31u, row = etid, tw = c.tw;
    const uint32_t rec = tile_record_bytes(tw, kPlanes);
    float* vt_all = reinterpret_cast<float*>(smem + p.sm_vt);
    float* vt = vt_all + row;      // this thread's accumulators: vt[n * kVtStride], token n
    uint32_t* arrive_mid = reinterpret_cast<uint32_t*>(buf + p.off_arrive) + (par * 2u + 1u) * p.tile_capacity;
    long long w_tfull = 0, w_l1 = 0, w_l2 = 0;
    const long long t_role = tc.clk();
    #pragma unroll 1
    for (uint32_t ti = 0; ti < c.ntasks; ++ti) {
        const uint32_t t = c.tasks[ti];
        const uint32_t type = t >> 28, e = (t >> 20) & 0xFF, mt = (t >> 8) & 0xFFF, j = t & 0xFF;
        const uint32_t acc = ti & 1u, use = (ti >> 1) & 1u;
        const uint32_t tile = udiv_small(c.mid_base[e], tw) + mt;
        const uint32_t left = c.exp_count[e] - mt * tw, nv = left < tw ? left : tw;
        // the rows' records (source rank, token, slot, top-k weight): the loader copied the tile's header into slot ti mod 4
        bool ok = cx.warp_wait(&c.meta_full[ti & 3u], (ti >> 2) & 1u, kErrWaitActsFull);
        ok = ok && tc.wait(&c.tmem_full[acc], use, kErrWaitTmemFull, w_tfull);
        const long long t_work = tc.clk();
        if (ok) {
            tc_fence_after();
            if (ti == 0u && etid == 0u) cx.sm_phase(kSmFirstMmaDone);
            uint32_t raw[kTileTokens];
            tmem_ld_32x32b_x16(c.tmem_base + ((ew * 32u) << 16) + acc * kWideTokens, raw);
            tmem_ld_wait();
            #pragma unroll
            for (int n = 0; n < kTileTokens; ++n) vt[n * kVtStride] = __uint_as_float(raw[n]);
            if (nv > kTileTokens) {
                tmem_ld_32x32b_x16(c.tmem_base + ((ew * 32u) << 16) + acc * kWideTokens + kTileTokens, raw);
                tmem_ld_wait();
                #pragma unroll
                for (int n = 0; n < kTileTokens; ++n) vt[(kTileTokens + n) * kVtStride] = __uint_as_float(raw[n]);
            }
            tc_fence_before();
            mbar_arrive(&c.tmem_empty[acc]);
        }
        if (bar_red_or(kBarEpi, kNumEpiThreads, !ok)) return;
        if (etid == 0u && ti > 0u) mbar_arrive(&c.meta_empty[(ti - 1u) & 3u]);      // every thread is past the previous task's records
        const RowMeta* meta = c.meta_ring[ti & 3u];
        const uint32_t np = (c.tasks2[ti] >> 16) & 0xFFu;
        if (np > 1u) {
            // this SM covered only part of the tile's K range: park the partial sums, count in, and let the last
            // contributor add the parts in SM order (a fixed order: the result does not depend on who arrives last)
            const uint32_t tix = c.tasks3[ti], cfirst = c.tasks2[ti] >> 24;
            float* red = reinterpret_cast<float*>(buf + p.off_red);
            constexpr size_t kSlot = 2u * kTileTokens * kTileRows;           // floats: room for 32 rows
            float* mine = red + (static_cast<size_t>(blockIdx.x) * 2u + type) * kSlot + row;
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) mine[n * kTileRows] = vt[n * kVtStride];
            bar_sync(kBarEpi, kNumEpiThreads);
            if (etid == 0) {
                uint32_t* cnt = reinterpret_cast<uint32_t*>(buf + p.off_cnt) + type * p.cnt_per_phase + tix;
                const uint32_t old = atom_acq_rel_gpu_add(cnt, 1u);
                if (old == np - 1u) *cnt = 0u;
                c.red_old = old;
            }
            bar_sync(kBarEpi, kNumEpiThreads);
            if (c.red_old != np - 1u) continue;
            #pragma unroll 1
            for (uint32_t n = 0; n < nv; ++n) {
                float sum = 0.f;
                #pragma unroll 1
                for (uint32_t pc0 = 0; pc0 < np; pc0 += 4) {
                    float part_v[4];
                    #pragma unroll
                    for (uint32_t d = 0; d < 4; ++d) {
                        part_v[d] = 0.f;
                        if (pc0 + d < np)
                            part_v[d] = __uint_as_float(ld_cg_u32(red + (static_cast<size_t>(cfirst + pc0 + d) * 2u + type) * kSlot + n * kTileRows + row));
                    }
                    #pragma unroll
                    for (uint32_t d = 0; d < 4; ++d) if (pc0 + d < np) sum += part_v[d];
                }
                vt[n * kVtStride] = sum;
            }
            bar_sync(kBarEpi, kNumEpiThreads);                    // the sums are read across threads below
        }

        if (type == 0u) {
            // ---- L1. Weight rows come in groups of 16 = 8 gate rows then the 8 matching up rows: 64 output columns per
            //      token. Thread (token n = t / 4, q = t % 4) takes the columns [16 k + 4 q, 16 k + 4 q + 4), k = 0..3, of
            //      its token from the accumulator tile in shared memory: all tokens at once, sixteen independent values
            //      per thread, whatever the number of rows.
            const uint32_t n = etid >> 2, q = etid & 3u;
            const bool live = n < nv;
            const float* vrow = vt_all + (live ? n : 0u) * kVtStride;
            const float wgt = meta[live ? n : 0u].weight;
            float o[16];
            #pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                const uint32_t base = 32u * k + 16u * (q >> 1) + 4u * (q & 1u);
                const float4 g4 = *reinterpret_cast<const float4*>(vrow + base), u4 = *reinterpret_cast<const float4*>(vrow + base + 8u);
                const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
                #pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    float gate = bf16_round(gs[i] * p.l1_scale), up = bf16_round(us[i] * p.l1_scale);
                    if (p.has_clamp) { gate = fminf(gate, p.clamp); up = fminf(fmaxf(up, -p.clamp), p.clamp); }
                    const float sig = p.fast_math ? __frcp_rn(1.0f + __expf(-gate)) : 1.0f / (1.0f + expf(-gate));
                    float av = gate * sig * up * wgt;
                    if constexpr (kVec == 16) av = __fdiv_rn(av, p.mid_gs);
                    o[4 * k + i] = av;
                }
            }
            // block maxima: a block of 16 columns is one k over the four q threads; a block of 32 columns is two k
            float am[4];
            #pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                float a = fmaxf(fmaxf(fabsf(o[4 * k]), fabsf(o[4 * k + 1])), fmaxf(fabsf(o[4 * k + 2]), fabsf(o[4 * k + 3])));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
                am[k] = a;
            }
            uint32_t sfw = 0u, packed[4];
            #pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                float amax = kVec == 32 ? fmaxf(am[k & 2u], am[(k & 2u) + 1u]) : am[k];
                amax = fmaxf(amax, 1e-30f);
                uint32_t sf_byte; float sc[4];
                if constexpr (kVec == 32) {
                    sf_byte = ceil_pow2_exp(__fdiv_rn(amax, 6.0f));
                    const float sf = __uint_as_float(sf_byte << 23);
                    #pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) sc[i] = __fdiv_rn(o[4 * k + i], sf);
                    if ((k & 1u) == 0u) sfw |= sf_byte << (4u * k);          // blocks 0 and 1 -> bytes 0 and 1
                } else {
                    sf_byte = cvt_e4m3x2(__fdiv_rn(amax, 6.0f), 0.f) & 0xFFu;
                    const float sf = e4m3_to_float(sf_byte);
                    #pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const float av = o[4 * k + i];
                        sc[i] = sf > 0.f ? __fdiv_rn(av, sf) : (av == 0.f ? 0.f : copysignf(6.0f, av));
                    }
                    sfw |= sf_byte << (8u * k);
                }
                packed[k] = cvt_e2m1x2(sc[0], sc[1]) | (cvt_e2m1x2(sc[2], sc[3]) << 8);
            }
            // the token's 32 output bytes = two 16 B chunks: chunk c holds k = 2c, 2c + 1, each as the 2-byte pieces of q = 0..3
            const uint32_t v01 = packed[0] | (packed[1] << 16), v23 = packed[2] | (packed[3] << 16);
            uint32_t w01[4], w23[4];
            #pragma unroll
            for (uint32_t d = 0; d < 4; ++d) {
                w01[d] = __shfl_sync(0xffffffffu, v01, (lane & ~3u) + d);
                w23[d] = __shfl_sync(0xffffffffu, v23, (lane & ~3u) + d);
            }
            {
                // into the intermediate tile's image: the chunks at their swizzled place in the record of their K unit, the
                // scale bytes into that record's slots; then one count into the tile's arrival word (thread 0's release
                // covers the stores the barrier ordered before it)
                uint8_t* img = buf + p.off_mid_tiles + static_cast<size_t>(tile) * p.mid_tile_bytes;
                if (live && q < 2u) {
                    const uint32_t* w = q == 0u ? w01 : w23;
                    const uint4 val = make_uint4((w[0] & 0xFFFFu) | (w[1] << 16), (w[2] & 0xFFFFu) | (w[3] << 16),
                                                 (w[0] >> 16) | (w[1] & 0xFFFF0000u), (w[2] >> 16) | (w[3] & 0xFFFF0000u));
                    const uint32_t ci = j * 2u + q;
                    *reinterpret_cast<uint4*>(img + (ci >> 3) * rec + sw128_off(n, ci & 7u)) = val;
                } else if (live && q == 2u) {
                    if constexpr (kVec == 16)
                        *reinterpret_cast<uint32_t*>(img + (j >> 2) * rec + tw * 128u + (j & 3u) * tw * 16u + n * 16u) = sfw;
                    else
                        *reinterpret_cast<uint16_t*>(img + (j >> 2) * rec + tw * 128u + ((j >> 1) & 1u) * tw * 16u + n * 16u + (j & 1u) * 2u) = static_cast<uint16_t>(sfw);
                }
                bar_sync(kBarEpi, kNumEpiThreads);
                if (etid == 0u) {
                    // The count needs a release, and under the weight flood a release takes microseconds: it is handed to
                    // the releasing warp through a queue in shared memory (done here only if that queue is full).
                    const uint32_t head = c.rel_head;
                    if (head - *reinterpret_cast<volatile uint32_t*>(&c.rel_tail) < kRelQueue) {
                        c.rel_q[head % kRelQueue] = tile;
                        c.rel_t[head % kRelQueue] = tc.clk();
                        __threadfence_block();
                        *reinterpret_cast<volatile uint32_t*>(&c.rel_head) = head + 1u;
                    } else {
                        fence_proxy_async_all();
                        red_release_gpu_add(arrive_mid + tile, 1u);
                    }
                }
            }
        } else {
            // ---- L2: bf16 rows back to the token's source rank, as flagged words: the combine there polls the data itself.
            //      A pair of lanes per 16 B chunk (8 weight rows of one token, read from the accumulator tile in shared
            //      memory): each lane stores one 16 B half of the chunk's flagged image, full 32 B sectors per instruction.
            #pragma unroll 1
            for (uint32_t idx = etid; idx < nv * 32u; idx += kNumEpiThreads) {
                const uint32_t n = idx >> 5, ch = (idx & 31u) >> 1;
                const float* v = vt_all + n * kVtStride + ch * 8u;
                const float4 lo = *reinterpret_cast<const float4*>(v), hi = *reinterpret_cast<const float4*>(v + 4);
                auto pack = [&](float x0, float x1) -> uint32_t {
                    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x0 * p.l2_scale))) |
                           (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x1 * p.l2_scale))) << 16);
                };
                const uint4 val = make_uint4(pack(lo.x, lo.y), pack(lo.z, lo.w), pack(hi.x, hi.y), pack(hi.z, hi.w));
                uint8_t* dst = cx.p.peer[meta[n].src] + p.off_comb +
                    ((static_cast<size_t>(meta[n].token) * p.topk + meta[n].slot) * p.H + j * kTileRows) * 4u + ch * 32u;
                st_ll_half(dst, val, c.epoch + 1u, idx & 1u);
            }
            bar_sync(kBarEpi, kNumEpiThreads);            // the accumulator tile is read across threads: nobody refills it before all are done
        }
        if (etid == 0u) {
            if (ti == 0u) cx.sm_phase(kSmFirstEpilogue);
            if (type == 0u) cx.sm_phase(kSmLastL1Epilogue);
        }
        if (type == 0u) w_l1 += tc.clk() - t_work; else w_l2 += tc.clk() - t_work;
    }
    if (etid == 0u) {
        // the releasing warp ends when it finds this entry
        uint32_t head = c.rel_head, spins = 0;
        while (head - *reinterpret_cast<volatile uint32_t*>(&c.rel_tail) >= kRelQueue && ++spins < 4000000u) { }
        c.rel_q[head % kRelQueue] = 0xFFFFFFFFu;
        __threadfence_block();
        *reinterpret_cast<volatile uint32_t*>(&c.rel_head) = head + 1u;
        tc.total(21, w_tfull); tc.total(22, tc.clk() - t_role); tc.total(23, w_l1); tc.total(24, w_l2);
    }
}

// The releasing warp: counts finished intermediate tiles in for the L1 epilogue (queue of tile numbers in shared memory,
// written by the epilogue's first thread after the barrier that follows the tile's stores). The release orders those
// stores, which the queue hand-off made visible to this warp, before the count.
__device__ void role_releaser(const Ctx& cx, const TileP p) {
    Ctl& c = cx.c;
    uint8_t* const buf = cx.buf; const uint32_t par = cx.par;
    const TileCtx tc{cx, (p.knobs & kKnobWaitProfile) != 0u};
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t* arrive_mid = reinterpret_cast<uint32_t*>(buf + p.off_arrive) + (par * 2u + 1u) * p.tile_capacity;
    uint32_t tail = 0, spins = 0;
    long long lat_sum = 0, lat_max = 0, busy = 0;
    // (the whole warp stays in this loop: lanes that left it would spin in the combine and take the issue slots of the lane that works here)
    for (;;) {
        uint32_t tile = 0xFFFFFFFEu;
        if (lane == 0) {
            if (*reinterpret_cast<volatile uint32_t*>(&c.rel_head) != tail) {
                __threadfence_block();
                tile = *reinterpret_cast<volatile uint32_t*>(&c.rel_q[tail % kRelQueue]);
                const long long t_q = *reinterpret_cast<volatile long long*>(&c.rel_t[tail % kRelQueue]);
                ++tail;
                *reinterpret_cast<volatile uint32_t*>(&c.rel_tail) = tail;
                if (tile != 0xFFFFFFFFu) {
                    const long long t0 = tc.clk();
                    fence_proxy_async_all();
                    red_release_gpu_add(arrive_mid + tile, 1u);
                    const long long t1 = tc.clk();
                    busy += t1 - t0; lat_sum += t1 - t_q; lat_max = lat_max > t1 - t_q ? lat_max : t1 - t_q;
                }
            } else if ((++spins & 0xFFFu) == 0u && (cx.aborted() || cx.expired())) {
                tile = 0xFFFFFFFFu;
            }
        }
        tile = __shfl_sync(0xffffffffu, tile, 0);
        if (tile == 0xFFFFFFFFu) break;
    }
    if (lane == 0) { tc.total(27, lat_sum); tc.total(28, lat_max); tc.total(29, busy); }
}

// ---- more than 16 received rows: the rows are sorted into tile images in global memory, one image per token tile
//      (16 or 32 rows) of an expert: the rows' records, then per streamed K unit the unit's 128 B of every row in the
//      tensor core's swizzled order and the unit's scale-word slots. Row f belongs to SM f mod G; one warp per row.
//      Every finished row counts into its tile's arrival word.
template <int kVec>
__device__ __forceinline__ void sort_rows_into_tiles(const Ctx& cx, const uint8_t* inp, uint32_t total, bool own_ok, uint32_t flag_rx, uint32_t warp, uint32_t lane) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    uint8_t* buf = cx.buf;
    const uint32_t bid = blockIdx.x, G = gridDim.x, par = cx.par;
    const uint32_t el = p.e_local;
    constexpr uint32_t kPlanes = kUnitK / (4 * kVec);
    // first tile of every expert: running sum of ceil(rows / tile rows), expert-major (the schedule derives the same numbers)
    const uint32_t cnt0 = lane < el ? c.exp_count[lane] : 0u, cnt1 = lane + 32 < el ? c.exp_count[lane + 32] : 0u;
    const uint32_t tw = __any_sync(0xffffffffu, cnt0 > kTileTokens || cnt1 > kTileTokens) ? kWideTokens : static_cast<uint32_t>(kTileTokens);
    const uint32_t rec = tile_record_bytes(tw, kPlanes);
    const uint32_t m0 = udiv_small(cnt0 + tw - 1u, tw), m1 = udiv_small(cnt1 + tw - 1u, tw);
    uint32_t i0 = m0, i1 = m1;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v0 = __shfl_up_sync(0xffffffffu, i0, o), v1 = __shfl_up_sync(0xffffffffu, i1, o);
        if (static_cast<int>(lane) >= o) { i0 += v0; i1 += v1; }
    }
    const uint32_t tbase0 = i0 - m0, tbase1 = __shfl_sync(0xffffffffu, i0, 31) + i1 - m1;
    const uint32_t per_row = p.rc_row_bytes / 16u, xq = p.x_row_bytes / 16u;
    uint32_t* arrive = reinterpret_cast<uint32_t*>(buf + p.off_arrive) + par * 2u * p.tile_capacity;
    // Records of this warp's first 32 rows that are own rows without an entry in the scout's list or in shared memory:
    // lane k fetches the record of the warp's k-th row, all in one memory round trip (the row's token index is in it).
    const uint32_t f_first = bid + (warp - 2u) * G, f_step = kFillWarps * G;
    uint4 my_rec = make_uint4(0u, 0u, 0u, 0u);
    bool my_rec_bad = false;
    if (cx.own_direct && !own_ok) {
        const uint32_t f = f_first + lane * f_step;
        if (f < total && f >= kMetaSmemRows) {
            uint32_t r = 0;
            while (r + 1 < static_cast<uint32_t>(p.R) && f >= c.rx_prefix[r + 1]) ++r;
            if (r == static_cast<uint32_t>(p.rank))
                my_rec_bad = !cx.ll_read(cx.rx_row(r, f - c.rx_prefix[r]) + 2u * (p.rx_row_bytes - 16), flag_rx, my_rec, kErrWaitDispatchFlag, r);
        }
    }
    uint32_t done_tiles[4];                                 // tiles of the rows written since the last release (one release per four rows)
    uint32_t ndone = 0, krow = 0;
    #pragma unroll 1
    for (uint32_t f = f_first; f < total; f += f_step, ++krow) {
        const uint32_t e = c.meta_e[f];
        // position among the expert's rows = rows of the same expert received before this one
        uint32_t n = 0;
        #pragma unroll 1
        for (uint32_t base = 0; base < f; base += 128) {
            const uint32_t idx = base + lane * 4u;
            const uint32_t w = *reinterpret_cast<const uint32_t*>(c.meta_e + idx);
            #pragma unroll
            for (uint32_t b = 0; b < 4; ++b) n += (idx + b < f && ((w >> (8u * b)) & 0xFFu) == e) ? 1u : 0u;
        }
        n = __reduce_add_sync(0xffffffffu, n);
        const uint32_t tb0 = __shfl_sync(0xffffffffu, tbase0, e & 31u), tb1 = __shfl_sync(0xffffffffu, tbase1, e & 31u);
        const uint32_t tile = (e < 32u ? tb0 : tb1) + udiv_small(n, tw), pos = n - udiv_small(n, tw) * tw;
        uint32_t r = 0;
        while (r + 1 < static_cast<uint32_t>(p.R) && f >= c.rx_prefix[r + 1]) ++r;
        const uint32_t i = f - c.rx_prefix[r];
        const bool own = cx.own_direct && r == static_cast<uint32_t>(p.rank);
        const uint8_t* xs = nullptr;
        const uint8_t* sf = nullptr;
        const uint8_t* row_src = nullptr;
        RowMeta own_m{0, 0, 0, 0.f};
        bool rec_bad = false;
        if (own) {
            // the row's record: from the scout's list, or (a batch too large for that list) from the receive pool, where the
            // dispatch left the records of the own rows without their payload
            if (own_ok) own_m = c.own_meta[i];
            else if (f < kMetaSmemRows) own_m = c.rx_meta[f];
            else {
                uint4 q = my_rec;
                bool qbad = my_rec_bad;
                if (krow >= 32u) {                                  // (beyond the prefetched records: fetch it now)
                    q = make_uint4(0u, 0u, 0u, 0u);
                    if (lane == 0) qbad = !cx.ll_read(cx.rx_row(r, i) + 2u * (p.rx_row_bytes - 16), flag_rx, q, kErrWaitDispatchFlag, r);
                }
                const uint32_t src_lane = krow < 32u ? krow : 0u;
                rec_bad = __shfl_sync(0xffffffffu, qbad ? 1u : 0u, src_lane) != 0u;
                own_m = RowMeta{0, static_cast<int32_t>(__shfl_sync(0xffffffffu, q.y, src_lane)), static_cast<int32_t>(__shfl_sync(0xffffffffu, q.z, src_lane)),
                                __uint_as_float(__shfl_sync(0xffffffffu, q.w, src_lane))};
            }
            const uint32_t tok = static_cast<uint32_t>(own_m.token);
            xs = inp + p.off_x + static_cast<size_t>(tok) * p.x_row_bytes;
            sf = inp + p.off_x_sf + static_cast<size_t>(tok) * p.x_sf_row_bytes;
        } else {
            row_src = cx.rx_row(r, i);
        }
        uint8_t* head = buf + p.off_token_tiles + static_cast<size_t>(tile) * p.token_tile_bytes;
        uint8_t* img = head + kWideTokens * 16u;
        bool bad = tile >= p.tile_capacity || __any_sync(0xffffffffu, rec_bad);
        // (chunk `per_row` of a received row is its record {expert, token, slot, top-k weight}: it becomes the row's
        //  record {source rank, token, slot, weight} in the tile's header)
        if (own && lane == 0 && !bad) {
            const RowMeta m = own_m;
            *reinterpret_cast<uint4*>(head + pos * 16u) = make_uint4(r, static_cast<uint32_t>(m.token), static_cast<uint32_t>(m.slot), __float_as_uint(m.weight));
        }
        const uint32_t nread = own ? per_row : per_row + 1u;
        #pragma unroll 1
        for (uint32_t base = lane; base < nread && !bad; base += 4 * 32) {
            uint4 v[4];
            if (own) {
                #pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t ci = base + u * 32;
                    if (ci < xq) v[u] = ld_cg_v4(xs + ci * 16u);
                    else if (ci < per_row) v[u] = ld_cg_v4(sf + (ci - xq) * 16u);
                }
            } else {
                uint32_t spins = 0;
                bool ok;
                do {
                    ok = true;
                    #pragma unroll
                    for (uint32_t u = 0; u < 4; ++u) {
                        const uint32_t ci = base + u * 32;
                        if (ci < nread) {
                            const uint4 a = ld_volatile_v4(row_src + ci * 32u), b = ld_volatile_v4(row_src + ci * 32u + 16u);
                            ok = ok && ll_valid(a, b, flag_rx);
                            v[u] = ll_data(a, b);
                        }
                    }
                    if (!ok && (++spins & 0x3Fu) == 0u) {
                        if (cx.aborted()) bad = true;
                        else if (cx.expired()) { cx.fail(kErrWaitDispatchFlag, r); bad = true; }
                    }
                } while (!ok && !bad);
            }
            #pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                const uint32_t ci = base + u * 32;
                if (ci >= nread || bad) continue;
                if (ci == per_row) {
                    *reinterpret_cast<uint4*>(head + pos * 16u) = make_uint4(r, v[u].y, v[u].z, v[u].w);
                } else if (ci < xq) {
                    *reinterpret_cast<uint4*>(img + (ci >> 3) * rec + sw128_off(pos, ci & 7u)) = v[u];
                } else {
                    // four scale words g .. g + 3 of the row: word g belongs to K unit g / planes, plane g % planes
                    const uint32_t g = (ci - xq) * 4u;
                    const uint32_t wv[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                    #pragma unroll
                    for (uint32_t k = 0; k < 4; ++k)
                        if ((g + k) * 4u < static_cast<uint32_t>(p.x_sf_row_bytes))
                            *reinterpret_cast<uint32_t*>(img + ((g + k) / kPlanes) * rec + tw * 128u + ((g + k) % kPlanes) * tw * 16u + pos * 16u) = wv[k];
                }
            }
        }
        const bool any_bad = __any_sync(0xffffffffu, bad);      // (also orders the lanes' stores before lane 0's fence)
        if (any_bad) break;
        // the rows' arrival counts: one release fence per four rows (under the weight flood a release takes microseconds),
        // then one relaxed count per row
        done_tiles[ndone & 3u] = tile;
        ++ndone;
        if ((ndone & 3u) == 0u || f + f_step >= total) {
            if (lane == 0) {
                fence_proxy_async_all();
                __threadfence();
                const uint32_t nrel = (ndone & 3u) == 0u ? 4u : (ndone & 3u);
                for (uint32_t k = 0; k < nrel; ++k) atomicAdd(arrive + done_tiles[k], 1u);
                cx.sm_phase(kSmRowsCached);
            }
            ndone = 0;
        }
    }
}

// ============================================================================================= schedule
// One warp derives this SM's task list from the per-expert row counts (16-token tiles of the active experts,
// expert-major: M of them). Returns M << 16 | number of tasks. Out of line on purpose: a spare warp runs it once on
// dummy counts while the SM waits for the dispatch, so that the real call finds its instructions in the SM's cache
// (executed cold, the instruction fetches of this code cost more than its arithmetic).
__device__ __noinline__ uint32_t build_schedule(const KParams& p, Ctl& c, const uint32_t* counts, uint32_t bid, uint32_t G, uint32_t lane) {
    const uint32_t el = p.e_local;
    const uint32_t c0 = lane < el ? counts[lane] : 0u, c1 = lane + 32 < el ? counts[lane + 32] : 0u;
    // rows per token tile: 16, or 32 when the launch works from tile images and an expert has more than 16 rows
    const uint32_t tw = (c.bulk != 0u && __any_sync(0xffffffffu, c0 > kTileTokens || c1 > kTileTokens)) ? kWideTokens : static_cast<uint32_t>(kTileTokens);
    const uint32_t sh = tw == kWideTokens ? 5u : 4u;
    const uint32_t m0 = (c0 + tw - 1u) >> sh, m1 = (c1 + tw - 1u) >> sh;
    uint32_t i0 = m0, i1 = m1;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v0 = __shfl_up_sync(0xffffffffu, i0, o), v1 = __shfl_up_sync(0xffffffffu, i1, o);
        if (static_cast<int>(lane) >= o) { i0 += v0; i1 += v1; }
    }
    const uint32_t tot0 = __shfl_sync(0xffffffffu, i0, 31), M = tot0 + __shfl_sync(0xffffffffu, i1, 31);
    const bool big = __any_sync(0xffffffffu, c0 > 8u || c1 > 8u);
    if (lane == 0) {
        const bool split = p.nab == 1 && !big;
        c.nab = split ? 2u : static_cast<uint32_t>(p.nab);
        c.act_stride = split ? p.act_bytes / 2u : p.act_bytes;
        c.atom_stride = split ? 8u * 128u : kTileTokens * 128u;
        c.sbo = split ? 0u : 1024u;
        c.tw = tw;
    }
    const uint32_t x0 = i0 - m0, x1 = tot0 + i1 - m1;
    if (lane < el) c.mid_base[lane] = x0 * tw;
    if (lane + 32 < el) c.mid_base[lane + 32] = x1 * tw;
    if (M <= kMaxMTiles) {
        #pragma unroll 1
        for (uint32_t mt = 0; mt < m0; ++mt) c.mtl[x0 + mt] = (lane << 16) | mt;
        #pragma unroll 1
        for (uint32_t mt = 0; mt < m1; ++mt) c.mtl[x1 + mt] = ((lane + 32) << 16) | mt;
    }
    __syncwarp();
    // A phase has NT = M * n weight-tile tasks of k units each. The first r = NT % G tiles are the remainder: tile t of
    // them is shared by the SMs [ceil(t G / r), ceil((t + 1) G / r)), each taking one contiguous range of the tile's K
    // units (sizes differ by at most one; parts are reduced by the last contributor). Every SM has at most one such
    // partial task per phase, and it runs first. Then SM g runs the whole tiles r + g, + G, ...
    // The two phases are worked out side by side: lanes 0..15 take phase 0 (L1), lanes 16..31 phase 1 (L2); the scalar
    // arithmetic of a phase is the same in its 16 lanes, the whole tiles are spread over them.
    uint32_t nmine = 0;
    if (M <= kMaxMTiles) {
        const uint32_t type = lane >> 4, l16 = lane & 15u;
        const uint32_t n = type ? p.n2_tiles : p.n1_tiles, k = type ? p.k2_units : p.k1_units;
        const uint32_t NT = M * n, r = NT - udiv_small(NT, G) * G;
        uint32_t has_split = 0u, s_t = 0u, s_word = 0u;
        if (r > 0u) {
            const uint32_t t = udiv_small(bid * r, G);
            const uint32_t gs = udiv_small(t * G + r - 1u, r), ge = udiv_small((t + 1u) * G + r - 1u, r);
            const uint32_t S = ge - gs, li = bid - gs, base = udiv_small(k, S), extra = k - base * S;
            const uint32_t ub = li * base + (li < extra ? li : extra), ue = ub + base + (li < extra ? 1u : 0u);
            has_split = ue > ub ? 1u : 0u;
            s_t = t;
            s_word = ub | (ue << 8) | ((S < k ? S : k) << 16) | (gs << 24);
        }
        const uint32_t first_whole = r + bid;
        const uint32_t nwhole = first_whole < NT ? udiv_small(NT - 1u - first_whole, G) + 1u : 0u;
        const uint32_t cnt_type = has_split + nwhole;
        const uint32_t cnt0 = __shfl_sync(0xffffffffu, cnt_type, 0), cnt1 = __shfl_sync(0xffffffffu, cnt_type, 16);
        const uint32_t basepos = type ? cnt0 : 0u;                 // the tasks of phase 0 come first
        if (l16 == 0u && has_split && basepos < kMaxTasks) {
            const uint32_t mi = udiv_small(s_t, n), ent = c.mtl[mi];
            c.tasks[basepos] = task_pack(type, ent >> 16, ent & 0xFFFFu, s_t - mi * n);
            c.tasks2[basepos] = s_word;
            c.tasks3[basepos] = s_t;
        }
        #pragma unroll 1
        for (uint32_t i = l16; i < nwhole; i += 16) {
            const uint32_t pos = basepos + has_split + i, t = first_whole + i * G;
            if (pos < kMaxTasks) {
                const uint32_t mi = udiv_small(t, n), ent = c.mtl[mi];
                c.tasks[pos] = task_pack(type, ent >> 16, ent & 0xFFFFu, t - mi * n);
                c.tasks2[pos] = (k << 8) | (1u << 16);
                c.tasks3[pos] = t;
            }
        }
        __syncwarp();
        if (lane == 0) c.n1_tasks = cnt0;
        nmine = cnt0 + cnt1;
    }    return (M << 16) | (nmine < 0xFFFFu ? nmine : 0xFFFFu);
}

// ============================================================================================= scout
// One warp per SM has nothing to do until the roles start. It (a) lists the routed rows of this rank's own tokens
// straight from topk_idx, so that no SM has to wait for the own-rank header line to learn them, and (b) watches the
// other ranks' header lines and records as they arrive; for every expert it learns to be live it asks for this SM's
// share of the expert's W1 and W2 units to be brought into the L2 (units u = SM, SM + G, ... of the expert's stream:
// all SMs together cover every byte once). The weight stream therefore starts when the first live expert is known,
// not when the last header has arrived and the schedule is built; the roles' bulk copies then find their units in the
// L2 or already on their way. The routing entries of the own tokens are loaded before the prologue's barrier.
struct ScoutRegs { long long tk[kOwnCap / 32]; float tw[kOwnCap / 32]; };

__device__ __forceinline__ void scout_load_own(const KParams& p, const uint8_t* inp, uint32_t lane, ScoutRegs& r) {
    const long long* tk = reinterpret_cast<const long long*>(inp + p.off_topk_idx);
    const float* tw = reinterpret_cast<const float*>(inp + p.off_topk_w);
    const uint32_t n = static_cast<uint32_t>(p.T) * p.topk;
    #pragma unroll
    for (uint32_t i = 0; i < kOwnCap / 32; ++i) {
        const uint32_t idx = i * 32 + lane;
        r.tk[i] = idx < n ? tk[idx] : -1ll;
        r.tw[i] = idx < n ? tw[idx] : 0.f;
    }
}

__device__ __forceinline__ uint64_t warp_or_u64(uint64_t v) {
    const uint32_t lo = __reduce_or_sync(0xffffffffu, static_cast<uint32_t>(v));
    const uint32_t hi = __reduce_or_sync(0xffffffffu, static_cast<uint32_t>(v >> 32));
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

struct ScoutState { uint64_t known; uint32_t asked; };

// this SM's share of the weights of the experts in `fresh`: W1 of all of them first (the L1 phase needs it first)
__device__ __forceinline__ void scout_ask(const Ctx& cx, ScoutState& st, uint64_t fresh, uint32_t lane, uint32_t G) {
    const KParams& p = cx.p;
    if ((p.knobs & kKnobPrefetch) == 0u || fresh == 0ull) return;
    const uint32_t bid = blockIdx.x;
    if (st.asked == 0u && lane == 0) { cx.note_first_weight_request(); }
    #pragma unroll 1
    for (uint32_t layer = 0; layer < 2; ++layer) {
        const uint32_t per = layer ? p.n2_tiles * p.k2_units : p.n1_tiles * p.k1_units;
        const uint32_t limit = layer ? p.pf_w2_max : p.pf_w1_max;
        const uint8_t* base = layer ? p.w2 : p.w1;
        uint64_t m = fresh;
        uint32_t n = st.asked;
        while (m != 0ull && n < limit) {
            const uint32_t e = static_cast<uint32_t>(__ffsll(static_cast<long long>(m))) - 1u;
            m &= m - 1ull;
            ++n;
            #pragma unroll 1
            for (uint32_t u = bid + lane * G; u < per; u += 32u * G)
                bulk_prefetch_l2(base + (static_cast<size_t>(e) * per + u) * p.unit_bytes, p.unit_bytes);
        }
    }
    st.asked += static_cast<uint32_t>(__popcll(fresh));
}

// Phase 1 (needs nothing of the prologue): list this rank's own routed rows from the routing entries the warp loaded
// at kernel entry, publish the list (named barrier kBarOwn: the scout arrives, the other warps wait there when they
// need the list), then ask for those experts' weights.
__device__ __noinline__ void scout_own_rows(const Ctx& cx, ScoutState& st, const ScoutRegs& reg, bool own_ok, uint32_t nthreads,
                                            uint32_t lane, uint32_t G) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    if (own_ok) {
        const uint32_t n = static_cast<uint32_t>(p.T) * p.topk;
        uint32_t cnt = 0;
        uint64_t m = 0ull;
        #pragma unroll
        for (uint32_t i = 0; i < kOwnCap / 32; ++i) {
            if (i * 32 < n) {
                const uint32_t idx = i * 32 + lane;
                const long long ex = reg.tk[i];
                const uint32_t ex32 = ex >= 0 && ex < 0x10000 ? static_cast<uint32_t>(ex) : 0u;
                const uint32_t dest = udiv_small(ex32, p.e_local), tok = udiv_small(idx, p.topk);
                const bool mine = idx < n && ex >= 0 && ex < 0x10000 && dest == static_cast<uint32_t>(p.rank);
                const uint32_t b = __ballot_sync(0xffffffffu, mine);
                if (mine) {
                    const uint32_t pos = cnt + __popc(b & ((1u << lane) - 1u)), el = ex32 - dest * p.e_local;
                    c.own_e[pos] = static_cast<uint8_t>(el);
                    c.own_meta[pos] = RowMeta{p.rank, static_cast<int32_t>(tok), static_cast<int32_t>(idx - tok * p.topk), reg.tw[i]};
                    m |= 1ull << (el & 63u);
                }
                cnt += __popc(b);
            }
        }
        if (lane == 0) { c.own_cnt = cnt; cx.sm_phase(kSmOwnListed); }
        st.known = warp_or_u64(m);
    }
    __threadfence_block();
    bar_arrive(kBarOwn, nthreads);
    scout_ask(cx, st, st.known, lane, G);
}

// Phase 2 (after the prologue: launch number and receive-pool parity are known): watch the other ranks' header lines and
// records arrive, asking for every newly seen expert's weights, until every source has been seen.
__device__ __noinline__ void scout_watch_peers(const Ctx& cx, ScoutState& st, bool own_ok, uint32_t lane, uint32_t G) {
    const KParams& p = cx.p; Ctl& c = cx.c;
    if ((p.knobs & kKnobPrefetch) == 0u) return;
    const uint32_t R = p.R, flag = c.epoch + 1u;
    uint32_t pending = (R >= 32u ? 0xFFFFFFFFu : (1u << R) - 1u);
    if (own_ok) pending &= ~(1u << p.rank);
    uint32_t passes = 0;
    while (pending != 0u) {
        uint64_t fresh = 0ull;
        #pragma unroll 1
        for (uint32_t r = 0; r < R; ++r) {
            if (((pending >> r) & 1u) == 0u) continue;
            const uint8_t* region = cx.buf + p.off_rx + static_cast<size_t>(cx.par * R + r) * p.rx_region;
            const uint4 ha = ld_volatile_v4(region), hb = ld_volatile_v4(region + 16);
            if (!ll_valid(ha, hb, flag)) continue;
            const uint32_t cnt = ha.x <= static_cast<uint32_t>(p.cap) ? ha.x : 0u;
            bool all = true;
            uint64_t m = 0ull;
            #pragma unroll 1
            for (uint32_t base = 0; base < cnt; base += 32) {
                const uint32_t i = base + lane;
                bool ok = true;
                if (i < cnt) {
                    const uint8_t* src = cx.rx_row(r, i) + 2u * (p.rx_row_bytes - 16);
                    const uint4 a = ld_volatile_v4(src), b = ld_volatile_v4(src + 16);
                    ok = ll_valid(a, b, flag);
                    // only experts this rank holds: the prefetch address must lie inside the weights
                    if (ok && (a.x & 0xFFu) < static_cast<uint32_t>(p.e_local)) m |= 1ull << (a.x & 63u);
                }
                all = __all_sync(0xffffffffu, ok) && all;
            }
            fresh |= warp_or_u64(m);
            if (all) pending &= ~(1u << r);
        }
        fresh &= ~st.known;
        // (once every source has been seen the other warps are about to fetch the received rows and to start the real
        // weight copies: a prefetch issued now would only stand in their way)
        if (pending != 0u) scout_ask(cx, st, fresh, lane, G);
        st.known |= fresh;
        if ((++passes & 0xFu) == 0u && (cx.aborted() || cx.expired())) break;   // the header wait of the other warps reports the failure
    }
}

// ============================================================================================= the kernel
template <int kVec, bool kUmma, bool kFe, bool kA8, bool kTiles>
__global__ void __launch_bounds__(kA8 ? kThreads + kNumExpThreads : kThreads, 1) mega_moe_kernel(const __grid_constant__ KParams p) {
    constexpr uint32_t kNT = kA8 ? kThreads + kNumExpThreads : kThreads;       // threads of this instantiation
    const unsigned long long t_first = globaltimer_ns();
    extern __shared__ uint8_t smem_raw[];
    __shared__ Ctl c;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, bid = blockIdx.x, G = gridDim.x;
    uint8_t* buf = p.peer[p.rank];
    const uint8_t* inp = kFe ? buf : p.inp;          // the fused frontend writes the input views itself (into the buffer)
    uint32_t* ctrl32 = reinterpret_cast<uint32_t*>(buf + p.off_ctrl);
    // the spare warp: the last one (it takes no part in the dispatch copies); with the fused frontend every warp is busy
    constexpr uint32_t kCopyWarps = kFe ? kNT / 32 : kNT / 32 - 1;
    constexpr bool kScout = !kFe;
    const bool own_ok = kScout && (p.knobs & kKnobOwnRows) != 0u && static_cast<uint32_t>(p.T) * p.topk <= kOwnCap &&
                        p.inp == buf;      // (inputs in mapped host memory are read by the dispatching SMs only)

    // ---- prologue
    constexpr uint32_t kO = kScout ? kNT - 32u : kNT;        // threads of the warps other than the scout
    const bool is_scout = kScout && warp == kCopyWarps;
    ScoutRegs sreg;
    ScoutState sst{0ull, 0u};
    if constexpr (kScout) {
        if (is_scout) {
            if (own_ok) scout_load_own(p, inp, lane, sreg);
            if (lane == 0) reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmWFirst)[bid] = ~0ull;
        }
    }
    if (tid == 0) {
        const uint32_t ep = ctrl32[kCtrlEpoch / 4 + bid];
        ctrl32[kCtrlEpoch / 4 + bid] = ep + 1u;
        c.epoch = ep; c.abort_flag = 0u; c.ntasks = 0u; c.dcount = 0u; c.comb_next = 0u; c.issued = 0u; c.decode = 0u; c.bulk = 0u; c.rel_head = 0u; c.rel_tail = 0u; c.rissued = 0u;
        if constexpr (!kScout) c.own_cnt = 0u;
        for (int s = 0; s < (p.nstage > static_cast<int>(p.nstage_wide) ? p.nstage : static_cast<int>(p.nstage_wide)); ++s) { mbar_init(&c.full[s], 1); mbar_init(&c.empty[s], kA8 ? kNumExpThreads / 64 : (kUmma ? 1 : kNumEpiThreads)); }
        #pragma unroll 1
        for (int i = 0; i < 2; ++i) {
            mbar_init(&c.acts_full[i], 1); mbar_init(&c.acts_empty[i], kUmma ? 1 : kNumEpiThreads);
            mbar_init(&c.tmem_full[i], 1); mbar_init(&c.tmem_empty[i], kNumEpiThreads);
            mbar_init(&c.xfull[i], kNumExpThreads / 64); mbar_init(&c.xempty[i], 1);
        }
        mbar_init(&c.tile_full, kFillWarps);
        mbar_fence_init();
        reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmEntry)[bid] = t_first;
        if constexpr (!kScout) reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmWFirst)[bid] = ~0ull;
    }
    if (kTiles && tid == 64) {
        // (the barriers only the tile-image roles use, set up by another thread than the one that does the rest)
        #pragma unroll 1
        for (uint32_t s2 = 0; s2 < p.nrec; ++s2) { mbar_init(&c.rfull[s2], 1); mbar_init(&c.rempty[s2], 1); }
        #pragma unroll 1
        for (int i = 0; i < 4; ++i) { mbar_init(&c.meta_full[i], 1); mbar_init(&c.meta_empty[i], 1); }
        mbar_fence_init();
    }
    // the token staging area starts from zero (the dispatch lists and the frontend's scratch that pass through it later
    // leave finite bytes; whatever sits in rows beyond a task's valid tokens only reaches accumulator columns nobody reads)
    if (!is_scout) {
        #pragma unroll 1
        for (uint32_t off = tid * 16u; off < p.stage_region; off += kO * 16u)
            *reinterpret_cast<uint4*>(smem + p.sm_act + off) = make_uint4(0, 0, 0, 0);
    }
    if (warp == 1) { tmem_alloc(&c.tmem_base, kTmemCols); tmem_relinquish(); tc_fence_before(); }
    if (tid < kMaxLocalExperts) c.exp_count[tid] = 0u;
    // Larger batches (the build with tile images): the rows of this rank's own tokens still get their header line and
    // records in the receive pool, but their payload does not travel: whoever needs such a row reads the token where the
    // caller put it (its index is in the record).
    const bool own_skip = kTiles && !kFe && !own_ok && p.inp == buf && static_cast<uint32_t>(p.T) * p.topk > kOwnCap;
    Ctx cx{p, c, buf, smem, globaltimer_ns() + p.timeout_ns, 0u, own_ok || own_skip};
    if (is_scout) {
        // the scout does not wait for the prologue: it lists the own rows and asks for their experts' weights first
        bar_arrive(kBarPrologue, kNT);
        scout_own_rows(cx, sst, sreg, own_ok, kNT, lane, G);
        bar_sync(kBarGo, kNT);
    } else {
        bar_sync(kBarPrologue, kNT);
        if constexpr (kScout) { __threadfence_block(); bar_arrive(kBarGo, kNT); }
    }
    tc_fence_after();
    cx.par = c.epoch & 1u;
    const uint32_t epoch = c.epoch, par = cx.par;
    const uint32_t ndisp = static_cast<uint32_t>(p.ndisp);
    // arrival counters of the operand tile images: this launch counts in the set of its parity and clears the other one
    // for the next launch (the launch before this one, which used that set, has ended)
    if (!is_scout) {
        uint32_t* other = reinterpret_cast<uint32_t*>(buf + p.off_arrive) + (par ^ 1u) * 2u * p.tile_capacity;
        #pragma unroll 1
        for (uint32_t i = bid * kO + tid; i < 2u * p.tile_capacity; i += G * kO) other[i] = 0u;
    }
    // The rows of this rank's own tokens never travel when `own_ok`: every SM lists them from topk_idx and reads their
    // tokens where the caller put them. The SM that would have dispatched them only leaves their header line and records
    // in the receive pool (its scout does, off the critical path), for whoever inspects the pool afterwards.
    const bool dispatching = bid < static_cast<uint32_t>(p.R) * ndisp &&
                             !(own_ok && bid - udiv_small(bid, p.R) * p.R == static_cast<uint32_t>(p.rank));

  if (is_scout) {
    if (own_ok && bid == static_cast<uint32_t>(p.rank)) {
        uint8_t* region = buf + p.off_rx + static_cast<size_t>(par * p.R + p.rank) * p.rx_region;
        const uint32_t cnt = c.own_cnt, flag = epoch + 1u;
        if (lane == 0) st_ll_16B(region, make_uint4(cnt, 0u, 0u, 0u), flag);
        #pragma unroll 1
        for (uint32_t i = lane; i < cnt; i += 32) {
            const RowMeta m = c.own_meta[i];
            st_ll_16B(region + 32u + static_cast<size_t>(i) * 2u * p.rx_row_bytes + 2u * (p.rx_row_bytes - 16),
                      make_uint4(c.own_e[i], static_cast<uint32_t>(m.token), static_cast<uint32_t>(m.slot), __float_as_uint(m.weight)), flag);
        }
    }
    scout_watch_peers(cx, sst, own_ok, lane, G);
    bar_sync(kBarSched, kNT);
  } else {
    if (bid == 0 && tid == 0) {
        ctrl32[kCtrlStatus / 4 + 1] = epoch + 1u;
        reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlStamps)[kStampEntry] = t_first;
        cx.stamp(kStampPrologue);
    }
    if (tid == 0) {
        reinterpret_cast<unsigned long long*>(buf + p.off_ctrl + kCtrlSmPhase)[bid * kSmPhaseSlots + kSmEntry] = t_first;
        cx.sm_phase(kSmPrologue);
    }
    // The control block and the split-tile counters are touched late, on the critical dependency chain, and by then
    // they have usually been evicted from the L2 by the weight stream of earlier work: ask for their lines now.
    if (warp == 6) {
        const uint32_t g = bid * 32 + lane, gn = G * 32;
        #pragma unroll 1
        for (uint32_t off = g * 128u; off < 8192u; off += gn * 128u) prefetch_l2_line(buf + p.off_ctrl + off);
        const size_t cnt_bytes = static_cast<size_t>(2) * p.cnt_per_phase * 4;
        #pragma unroll 1
        for (size_t off = static_cast<size_t>(g) * 128u; off < (cnt_bytes < 65536 ? cnt_bytes : 65536); off += gn * 128u) prefetch_l2_line(buf + p.off_cnt + off);
    }

    if constexpr (!kFe) {
        if ((p.knobs & kKnobRehearse) != 0u && !dispatching && (warp == 2 || warp == 3)) role_stager(cx, warp - 2, lane, true);
    }

    // ---- warm-up of the scheduler's instructions: on the SMs that do not dispatch, warp 6 is idle until the roles start,
    //      so it runs the scheduler once on dummy counts (eight experts with one row). The real call, which sits on the
    //      critical path right after the dispatch arrives, then finds its instructions cached and overwrites everything
    //      this writes. (On the dispatching SMs warp 6 copies rows; their schedule runs cold.)
    if constexpr (!kFe) {
        if (warp == 6 && !dispatching && (p.R > 1 || !own_ok)) {       // (one rank with own rows listed: nothing to hide it behind)
            for (uint32_t e = lane; e < kMaxLocalExperts; e += 32) c.dry_count[e] = e < 8u ? 1u : 0u;
            __syncwarp();
            build_schedule(p, c, c.dry_count, bid, G, lane);
        }
    }

    // ---- router frontend (optional): all SMs compute partial logits (one memory round trip per item) and publish them
    //      as flagged records; the dispatching SMs poll the records of a token, select its top-8 and weights. No barrier
    //      and no arrival counter in between: the selecting warps wait for exactly the values they read.
    if constexpr (kFe) {
        const uint32_t fe_flag = epoch + 1u;
        fe_logits_items(p.fe, bid * (kNT / 32) + warp, G * (kNT / 32), lane, fe_flag);
        if (dispatching) {                       // (every dispatching SM selects all tokens: it needs the whole routing for its row list)
            float* sc = reinterpret_cast<float*>(smem + p.sm_act) + warp * 2 * p.fe.E;
            auto give_up = [&]() -> bool {
                if (cx.aborted()) return true;
                if (cx.expired()) { cx.fail(kErrWaitFrontend); return true; }
                return false;
            };
            #pragma unroll 1
            for (uint32_t t = warp; t < static_cast<uint32_t>(p.T); t += kNT / 32) {
                const bool nz = fe_row_nonzero(p.fe.hidden + static_cast<size_t>(t) * p.H, p.H, lane);
                if (!fe_select_token(p.fe, t, sc, nz, lane, fe_flag, give_up)) break;
            }
            __threadfence();                 // the routing written above is read by other SMs of this launch (combine)
            bar_sync(kBarMain, kO);
        }
        if (bid == 0 && tid == 0) cx.stamp(kStampFrontend);
    }

    // ---- dispatch: the SMs d, d + R, d + 2R, ... (`ndisp` of them: one at decode sizes, more when a destination gets many
    //      rows) push this rank's rows for rank d; each builds the same row list and takes the rows i = part (mod ndisp)
    if (dispatching && warp < kCopyWarps) {
        const uint32_t part = udiv_small(bid, p.R), d = bid - part * p.R;
        uint32_t* dlist = reinterpret_cast<uint32_t*>(smem + p.sm_act);
        if (warp == 0) {
            const long long* tk = reinterpret_cast<const long long*>(inp + p.off_topk_idx);
            const uint32_t n = static_cast<uint32_t>(p.T) * p.topk;
            uint32_t cnt = 0;
            constexpr uint32_t kDl = kTiles ? 4u : 1u;             // (large batches: four loads in flight, one memory round trip per 128 routing entries)
            #pragma unroll 1
            for (uint32_t base0 = 0; base0 < n; base0 += kDl * 32) {
                long long exs[kDl];
                #pragma unroll
                for (uint32_t u = 0; u < kDl; ++u) {
                    const uint32_t i = base0 + u * 32 + lane;
                    exs[u] = i < n ? tk[i] : -1;
                }
                #pragma unroll
                for (uint32_t u = 0; u < kDl; ++u) {
                    const uint32_t i = base0 + u * 32 + lane;
                    const long long ex = exs[u];
                    const uint32_t ex32 = ex >= 0 && ex < 0x10000 ? static_cast<uint32_t>(ex) : 0u;
                    const uint32_t dest = udiv_small(ex32, p.e_local), tok = udiv_small(i, p.topk);
                    const bool m = ex >= 0 && ex < 0x10000 && dest == d;
                    const uint32_t b = __ballot_sync(0xffffffffu, m);
                    if (m) dlist[cnt + __popc(b & ((1u << lane) - 1u))] = (tok << 16) | ((i - tok * p.topk) << 8) | (ex32 - dest * p.e_local);
                    cnt += __popc(b);
                }
            }
            if (lane == 0) c.dcount = cnt;
        }
        bar_sync(kBarCopy, kCopyWarps * 32);
        const uint32_t cnt = c.dcount;
        const uint32_t nchunk = (p.rx_row_bytes - 16) / 16, xq = p.x_row_bytes / 16;      // payload chunks of a row: tokens, then scale bytes
        const uint32_t flag = epoch + 1u;
        uint8_t* region = p.peer[d] + p.off_rx + static_cast<size_t>(par * p.R + p.rank) * p.rx_region;
        uint8_t* dst_base = region + 32u;
        const float* tw = reinterpret_cast<const float*>(inp + p.off_topk_w);
        // Header line (row count) and the rows' 16 B records (expert, token, slot, weight) leave first: they are all the
        // receiver's scheduler needs, and they do not depend on the token data. Every word is self-validating (flagged),
        // so nothing has to order these stores against the payload that follows.
        if (tid == 0 && part == 0u) st_ll_16B(region, make_uint4(cnt, 0u, 0u, 0u), flag);
        #pragma unroll 1
        for (uint32_t i = part + tid * ndisp; i < cnt; i += kCopyWarps * 32 * ndisp) {
            const uint32_t ent = dlist[i], tok = ent >> 16, slot = (ent >> 8) & 0xFFu;
            st_ll_16B(dst_base + static_cast<size_t>(i) * 2u * p.rx_row_bytes + 2u * (p.rx_row_bytes - 16),
                      make_uint4(ent & 0xFFu, tok, slot, __float_as_uint(tw[tok * p.topk + slot])), flag);
        }
        if constexpr (kFe) {
            // quantise the tokens this SM sends: into the x / x_sf views (the same bytes whichever SM writes them) and, from
            // the same registers, into the destination's receive pool
            #pragma unroll 1
            for (uint32_t i = part + warp * ndisp; i < cnt; i += kCopyWarps * ndisp) {
                const uint32_t tok = dlist[i] >> 16;
                fe_quant_token(p.fe.hidden + static_cast<size_t>(tok) * p.H, p.H, kA8 ? 2 : (kVec == 32 ? 0 : 1), p.fe.x_gs,
                               buf + p.off_x + static_cast<size_t>(tok) * p.x_row_bytes,
                               buf + p.off_x_sf + static_cast<size_t>(tok) * p.x_sf_row_bytes, lane,
                               dst_base + static_cast<size_t>(i) * 2u * p.rx_row_bytes, flag, static_cast<uint32_t>(p.x_row_bytes));
            }
        } else if (!(own_skip && d == static_cast<uint32_t>(p.rank))) {
        // warp w copies rows w, w + 8, ...: lane l moves chunks l, l + 32, ... (eight in flight: one memory round trip for
        // a row of up to 4 KB)
        #pragma unroll 1
        for (uint32_t i = part + warp * ndisp; i < cnt; i += kCopyWarps * ndisp) {
            const uint32_t tok = dlist[i] >> 16;
            const uint8_t* xs_src = inp + p.off_x + static_cast<size_t>(tok) * p.x_row_bytes;
            const uint8_t* sf_src = inp + p.off_x_sf + static_cast<size_t>(tok) * p.x_sf_row_bytes;
            uint8_t* dst = dst_base + static_cast<size_t>(i) * 2u * p.rx_row_bytes;
            // a pair of lanes per 16 B payload chunk: each stores one 16 B half of its 32 B flagged image, so that a warp
            // instruction writes 512 contiguous bytes in full sectors (the packets that cross NVLink)
            #pragma unroll 1
            for (uint32_t base = lane; base < 2u * nchunk; base += 8 * 32) {
                uint4 v[8];
                #pragma unroll
                for (uint32_t u = 0; u < 8; ++u) {
                    const uint32_t ci = (base + u * 32) >> 1;
                    if (ci < xq) v[u] = *reinterpret_cast<const uint4*>(xs_src + ci * 16u);
                    else if (ci < nchunk) v[u] = *reinterpret_cast<const uint4*>(sf_src + (ci - xq) * 16u);
                }
                #pragma unroll
                for (uint32_t u = 0; u < 8; ++u) {
                    const uint32_t hc = base + u * 32, ci = hc >> 1;
                    if (ci < nchunk) st_ll_half(dst + ci * 32u, v[u], flag, hc & 1u);
                }
            }
        }
        }
        bar_sync(kBarCopy, kCopyWarps * 32);
    }
    if (bid == 0 && tid == 0) cx.stamp(kStampDispatched);

    // ---- receive: wait for every source rank's header line, then scan the received rows' records. The first 32 records
    //      of the first sources are fetched speculatively in the same memory round trip as the headers (thread 32 r + i
    //      takes record i of source r); a record that was not there yet, and any other record, is polled afterwards.
    //      The rows of this rank's own tokens need no header: the scout lists them from topk_idx (`own_ok`).
    const uint32_t flag_rx = epoch + 1u;
    const uint32_t spec_r = tid >> 5, spec_i = tid & 31u;
    constexpr uint32_t kSpecSources = kO / 32u;                       // sources whose first records have a speculating thread
    const bool spec = spec_r < static_cast<uint32_t>(p.R) && spec_r < kSpecSources && spec_i < static_cast<uint32_t>(p.cap) &&
                      !(own_ok && spec_r == static_cast<uint32_t>(p.rank));
    uint4 spec_a = make_uint4(0u, 0u, 0u, 0u), spec_b = spec_a;
    if (spec) {
        const uint8_t* src = cx.rx_row(spec_r, spec_i) + 2u * (p.rx_row_bytes - 16);
        spec_a = ld_volatile_v4(src); spec_b = ld_volatile_v4(src + 16);
    }
    if (tid < static_cast<uint32_t>(p.R) && !(own_ok && tid == static_cast<uint32_t>(p.rank))) {
        uint4 h = make_uint4(0u, 0u, 0u, 0u);
        cx.ll_read(buf + p.off_rx + static_cast<size_t>(par * p.R + tid) * p.rx_region, flag_rx, h, kErrWaitDispatchFlag, tid);
        c.rx_count[tid] = h.x <= static_cast<uint32_t>(p.cap) ? h.x : 0u;
    }
    if constexpr (kScout) bar_sync(kBarOwn, kNT);          // (all other warps + the scout's arrival: its list is written)
    else bar_sync(kBarMain, kO);
    if constexpr (kFe) __threadfence();
    uint32_t total = 0;
    {
        uint32_t pre[kMaxRanks + 1];
        #pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            pre[r] = total;
            if (r < p.R) total += (own_ok && r == p.rank) ? c.own_cnt : c.rx_count[r];
        }
        pre[kMaxRanks] = total;
        if (tid <= static_cast<uint32_t>(p.R)) c.rx_prefix[tid] = tid < static_cast<uint32_t>(p.R) ? pre[tid] : total;
        if (tid == 0) {
            if (total > kMetaCap) cx.fail(kErrMetaCapacity, total >> 4);
            if (bid == 0) cx.stamp(kStampFlagsSeen);
            cx.sm_phase(kSmCountsKnown);
            c.decode = (kUmma && !kA8 && p.rc_rows != 0u && total != 0u && total <= kTileTokens) ? 1u : 0u;     // (the cross-check engine reads the per-task staging buffers)
            c.bulk = (kTiles && kUmma && !kA8 && (p.knobs & kKnobTileImages) != 0u && p.nstage_wide >= 3u && p.nrec >= 2u && total > kTileTokens && total <= kMetaCap) ? 1u : 0u;
        }
        if (total <= kMetaCap) {
            auto take = [&](uint32_t f, const uint4& m) {
                const uint32_t e = m.x & 0xFFu;
                c.meta_e[f] = static_cast<uint8_t>(e);
                if (f < kMetaSmemRows) c.rx_meta[f] = RowMeta{0, static_cast<int32_t>(m.y), static_cast<int32_t>(m.z), __uint_as_float(m.w)};
                atomicAdd(&c.exp_count[e < kMaxLocalExperts ? e : 0], 1u);
            };
            const uint32_t spec_cnt = spec ? c.rx_count[spec_r] : 0u;
            if (spec && spec_i < spec_cnt) {
                uint4 m = ll_data(spec_a, spec_b);
                if (!ll_valid(spec_a, spec_b, flag_rx))
                    cx.ll_read(cx.rx_row(spec_r, spec_i) + 2u * (p.rx_row_bytes - 16), flag_rx, m, kErrWaitDispatchFlag, spec_r);
                take(pre[spec_r] + spec_i, m);
            }
            if (!kTiles || total <= kO) {
                // one record per thread and pass
                #pragma unroll 1
                for (uint32_t f = tid; f < total; f += kO) {
                    uint32_t r = 0;
                    #pragma unroll
                    for (int q = 1; q < kMaxRanks; ++q) r += (q < p.R && f >= pre[q]) ? 1u : 0u;
                    const uint32_t i = f - pre[r];
                    if (own_ok && r == static_cast<uint32_t>(p.rank)) {
                        const RowMeta om = c.own_meta[i];
                        take(f, make_uint4(c.own_e[i], static_cast<uint32_t>(om.token), static_cast<uint32_t>(om.slot), __float_as_uint(om.weight)));
                    } else if (!(i < 32u && r < kSpecSources)) {         // (else: taken by the speculative read above)
                        uint4 m = make_uint4(0u, 0u, 0u, 0u);
                        cx.ll_read(cx.rx_row(r, i) + 2u * (p.rx_row_bytes - 16), flag_rx, m, kErrWaitDispatchFlag, r);
                        take(f, m);
                    }
                }
            } else
            // (four records per thread in flight together: one memory round trip per four records of a large batch)
            #pragma unroll 1
            for (uint32_t f0 = tid; f0 < total; f0 += 4u * kO) {
                const uint8_t* src[4];
                uint4 ra[4], rb[4];
                uint32_t rr[4];
                #pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t f = f0 + u * kO;
                    src[u] = nullptr;
                    rr[u] = 0u;
                    if (f >= total) continue;
                    uint32_t r = 0;
                    #pragma unroll
                    for (int q = 1; q < kMaxRanks; ++q) r += (q < p.R && f >= pre[q]) ? 1u : 0u;
                    const uint32_t i = f - pre[r];
                    if (own_ok && r == static_cast<uint32_t>(p.rank)) {
                        const RowMeta om = c.own_meta[i];
                        take(f, make_uint4(c.own_e[i], static_cast<uint32_t>(om.token), static_cast<uint32_t>(om.slot), __float_as_uint(om.weight)));
                        continue;
                    }
                    if (i < 32u && r < kSpecSources) continue;           // taken by the speculative read above
                    src[u] = cx.rx_row(r, i) + 2u * (p.rx_row_bytes - 16);
                    rr[u] = r;
                    ra[u] = ld_volatile_v4(src[u]); rb[u] = ld_volatile_v4(src[u] + 16);
                }
                #pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    if (src[u] == nullptr) continue;
                    uint4 m = ll_data(ra[u], rb[u]);
                    if (!ll_valid(ra[u], rb[u], flag_rx)) cx.ll_read(src[u], flag_rx, m, kErrWaitDispatchFlag, rr[u]);
                    take(f0 + u * kO, m);
                }
            }
        }
    }
    bar_sync(kBarMain, kO);

    // ---- the rows received from other ranks go into the row cache (one warp per row, warps 2..6) while warp 0 builds the
    //      schedule and then starts the weight stream without waiting for them: these warps' roles (token staging,
    //      epilogue) are not needed before the first weights have landed, and the rows' payload may still be on its way
    //      (a sender pushes its header line and records first). The loads are in flight before the bulk copies of the
    //      weight stream start, which would otherwise make them wait behind megabytes.
    const bool is_ctl = warp < 2u;                       // warps 0 and 1 build the schedule and start the weight stream
    // ---- more than 16 received rows: the rows are sorted into tile images in global memory (see sort_rows_into_tiles)
    if (warp >= 2u && warp < 2u + kFillWarps && c.bulk != 0u && !cx.aborted()) {
        if constexpr (kTiles && kUmma && !kA8) sort_rows_into_tiles<kVec>(cx, inp, total, own_ok, flag_rx, warp, lane);
    }
    if (warp >= 2u && warp < 2u + kFillWarps && p.rc_rows != 0u && total <= kMetaCap && c.bulk == 0u && !cx.aborted()) {
        const bool decode = c.decode != 0u;
        const uint32_t per_row = p.rc_row_bytes / 16u, xq = p.x_row_bytes / 16u;
        const uint32_t limit = total < p.rc_rows ? total : p.rc_rows;
        const uint32_t my_e = lane < total ? c.meta_e[lane] : 0xFFu;      // (decode mode: at most 16 rows, one per lane)
        uint8_t* region = cx.tok_region();
        #pragma unroll 1
        for (uint32_t f = warp - 2u; f < limit; f += kFillWarps) {
            uint32_t r = 0;
            while (r + 1 < static_cast<uint32_t>(p.R) && f >= c.rx_prefix[r + 1]) ++r;
            const uint32_t i = f - c.rx_prefix[r];
            const bool own = cx.own_direct && r == static_cast<uint32_t>(p.rank);  // this rank's own token: read it where the caller put it
            // decode mode: row position in the shared tile = rows of experts with a smaller index, then the earlier rows
            // of the same expert (receive order)
            const uint32_t e = c.meta_e[f];
            const uint32_t pos = __popc(__ballot_sync(0xffffffffu, my_e < e)) +
                                 __popc(__ballot_sync(0xffffffffu, my_e == e) & ((1u << f) - 1u));
            const uint8_t* xs = nullptr;
            const uint8_t* sf = nullptr;
            const uint8_t* row_src = nullptr;
            if (own) {
                const uint32_t tok = static_cast<uint32_t>(own_ok ? c.own_meta[i].token : c.rx_meta[f].token);   // (f < 16: its record is in shared memory)
                xs = inp + p.off_x + static_cast<size_t>(tok) * p.x_row_bytes;
                sf = inp + p.off_x_sf + static_cast<size_t>(tok) * p.x_sf_row_bytes;
            } else {
                row_src = cx.rx_row(r, i);
            }
            uint8_t* raw_dst = region + f * p.rc_row_bytes;
            bool bad = false;
            #pragma unroll 1
            for (uint32_t base = lane; base < per_row && !bad; base += 4 * 32) {
                uint4 v[4];
                if (own) {
                    #pragma unroll
                    for (uint32_t u = 0; u < 4; ++u) {
                        const uint32_t ci = base + u * 32;
                        if (ci < xq) v[u] = ld_cg_v4(xs + ci * 16u);
                        else if (ci < per_row) v[u] = ld_cg_v4(sf + (ci - xq) * 16u);
                    }
                } else {
                    uint32_t spins = 0;
                    bool ok;
                    do {
                        ok = true;
                        #pragma unroll
                        for (uint32_t u = 0; u < 4; ++u) {
                            const uint32_t ci = base + u * 32;
                            if (ci < per_row) {
                                const uint4 a = ld_volatile_v4(row_src + ci * 32u), b = ld_volatile_v4(row_src + ci * 32u + 16u);
                                ok = ok && ll_valid(a, b, flag_rx);
                                v[u] = ll_data(a, b);
                            }
                        }
                        if (!ok && (++spins & 0x3Fu) == 0u) {
                            if (cx.aborted()) bad = true;
                            else if (cx.expired()) { cx.fail(kErrWaitDispatchFlag, r); bad = true; }
                        }
                    } while (!ok && !bad);
                }
                #pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t ci = base + u * 32;
                    if (ci >= per_row || bad) continue;
                    if (!decode) {
                        *reinterpret_cast<uint4*>(raw_dst + ci * 16u) = v[u];
                    } else if (ci < xq) {
                        *reinterpret_cast<uint4*>(region + (ci >> 3) * (kTileTokens * 128u) + sw128_off(pos, ci & 7u)) = v[u];
                    } else {
                        uint8_t* dst = cx.tile_asf() + (ci - xq) * 4u * 256u + pos * 16u;
                        *reinterpret_cast<uint32_t*>(dst) = v[u].x;
                        *reinterpret_cast<uint32_t*>(dst + 256u) = v[u].y;
                        *reinterpret_cast<uint32_t*>(dst + 512u) = v[u].z;
                        *reinterpret_cast<uint32_t*>(dst + 768u) = v[u].w;
                    }
                }
            }
            if (lane == 0) cx.sm_phase(kSmRowsCached);
        }
        if (decode) {
            fence_proxy_async_smem();                     // the tensor core reads the tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&c.tile_full);
        }
    }

    // ---- schedule. 16-token tiles of the active experts, expert-major: M of them. Every SM derives its own task list
    //      (L1 tasks, then L2 tasks) in closed form from the per-expert counts. Warps 0 and 1 publish it on kBarSched
    //      without waiting there; every other warp (the scout included) waits on that barrier before it takes up its role.
    if (is_ctl) {
        if (warp == 0 && !cx.aborted()) {
            const uint32_t res = build_schedule(p, c, c.exp_count, bid, G, lane);
            const uint32_t M = res >> 16, nmine = res & 0xFFFFu;
            const uint32_t nt1 = M * p.n1_tiles, nt2 = M * p.n2_tiles;
            if (lane == 0) {
                if (bid == 0) ctrl32[kCtrlStatus / 4 + 2] = c.bulk != 0u ? c.tw : 0u;      // (for whoever inspects the intermediate rows afterwards)
                c.nt1 = nt1; c.nt2 = nt2;
                if (M > kMaxMTiles || nmine > kMaxTasks) cx.fail(kErrTaskCapacity, nmine);
                else c.ntasks = nmine;
            }
        }
        bar_sync(kBarPost, 64);
        __threadfence_block();
        bar_arrive(kBarSched, kNT);
        if (bid == 0 && tid == 0) cx.stamp(kStampScheduled);
        if (tid == 0) { cx.stamp_max(kStampLastScheduled, globaltimer_ns()); cx.sm_phase(kSmScheduled); }
        if (bid == 0 && tid < static_cast<uint32_t>(p.e_local) && p.stats != nullptr && !cx.aborted())
            p.stats[tid] += static_cast<int>(c.exp_count[tid]);
    } else {
        bar_sync(kBarSched, kNT);
    }
  }

    // ---- roles
    bool tiles = false;
    if constexpr (kTiles && kUmma && !kA8) tiles = c.bulk != 0u;
    if (!cx.aborted() && tiles) {
        if constexpr (kTiles && kUmma && !kA8) {                     // (launches with more than 16 received rows)
            const TileP tp = make_tile_params(p);
            if (warp == 0) role_loader_tiles(cx, tp);
            else if (warp == 1) role_mma_tiles<kVec>(cx, tp, lane);
            else if (warp == 2) role_record_loader(cx, tp, kUnitK / (4 * kVec));
            else if (warp == 3) role_releaser(cx, tp);
            else if (warp >= 4 && warp < 8) role_epilogue_tiles<kVec>(cx, tp, tid - 128);
        }
    } else if (!cx.aborted()) {
        if (warp == 0) role_loader(cx);
        else if (warp == 1) { if constexpr (kUmma) role_mma<kVec, kA8>(cx, lane); }
        else if (warp < 4) role_stager(cx, warp - 2, lane, false);
        else if (warp < 8) role_epilogue<kVec, kUmma, kA8>(cx, tid - 128);
        else { if constexpr (kA8) role_expander(cx, tid - kThreads); }
    }
    const bool early = (p.knobs & kKnobEarlyCombine) != 0u;
    if (!early) __syncthreads();
    if (tid == 128) {                                   // first epilogue thread: this SM's tasks are finished
        if (bid == 0) cx.stamp(kStampTasksDone);
        cx.stamp_max(kStampLastTasksDone, globaltimer_ns());
        cx.sm_phase(kSmTasksDone);
    }

    // ---- combine. No grid-wide or cross-rank barrier precedes it: the expert outputs arrive as flagged words and every
    //      thread polls exactly the words it sums. Item = (token, 16 B chunk of the row); the items b, b + G, ... belong
    //      to SM b (a small batch uses the whole GPU) and its threads take them one by one. A warp comes here as soon as
    //      its role has ended, so the first polls (and the first execution of this code) overlap the SM's last tasks.
    if (!cx.aborted()) {
        const uint32_t chunks_per_row = p.H / 8, nitems = static_cast<uint32_t>(p.T) * chunks_per_row;
        const long long* tk = reinterpret_cast<const long long*>(inp + p.off_topk_idx);
        const uint32_t flag = epoch + 1u;
        const size_t sstride = static_cast<size_t>(p.H) * 4u;
        bool bad = false;
        uint32_t static_k = tid;
        #pragma unroll 1
        while (!bad) {
            uint32_t k;
            if (early) k = atomicAdd(&c.comb_next, 1u); else { k = static_k; static_k += kNT; }
            const uint32_t idx = bid + k * G;
            if (k >= nitems || idx >= nitems) break;
            const uint32_t tok = udiv_small(idx, chunks_per_row), ch = idx - tok * chunks_per_row;
            uint32_t mask = 0u;
            for (int sl = 0; sl < p.topk; ++sl) {
                long long ex;
                if constexpr (kFe) ex = static_cast<long long>(ld_volatile_u64(tk + tok * p.topk + sl)); else ex = tk[tok * p.topk + sl];
                mask |= (ex >= 0 ? 1u : 0u) << sl;
            }
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const uint8_t* cbase = buf + p.off_comb + (static_cast<size_t>(tok) * p.topk * p.H) * 4u + ch * 32u;
            #pragma unroll 1
            for (int s0 = 0; s0 < p.topk && !bad; s0 += 8) {
                // eight routes' words in flight, re-read until each live route carries this launch's flag; a masked route
                // contributes +0.0, which leaves the running sums bit-identical; routes are added in slot order
                uint4 v[8];
                uint32_t spins = 0;
                bool ok;
                do {
                    ok = true;
                    #pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        v[u] = make_uint4(0u, 0u, 0u, 0u);
                        if ((mask >> (s0 + u)) & 1u) {
                            const uint8_t* src = cbase + static_cast<size_t>(s0 + u) * sstride;
                            const uint4 a = ld_volatile_v4(src), b = ld_volatile_v4(src + 16);
                            ok = ok && ll_valid(a, b, flag);
                            v[u] = ll_data(a, b);
                        }
                    }
                    if (!ok && (++spins & 0x3Fu) == 0u) {
                        if (cx.aborted()) bad = true;
                        else if (cx.expired()) { cx.fail(kErrWaitCombineFlag, tok); bad = true; }
                    }
                } while (!ok && !bad);
                #pragma unroll
                for (int u = 0; u < 8; ++u) {
                    acc[0] += __uint_as_float(v[u].x << 16); acc[1] += __uint_as_float(v[u].x & 0xFFFF0000u);
                    acc[2] += __uint_as_float(v[u].y << 16); acc[3] += __uint_as_float(v[u].y & 0xFFFF0000u);
                    acc[4] += __uint_as_float(v[u].z << 16); acc[5] += __uint_as_float(v[u].z & 0xFFFF0000u);
                    acc[6] += __uint_as_float(v[u].w << 16); acc[7] += __uint_as_float(v[u].w & 0xFFFF0000u);
                }
            }
            if (bad) break;
            uint4 o;
            uint32_t* ow = &o.x;
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * q]));
                const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * q + 1]));
                ow[q] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.y) + (static_cast<size_t>(tok) * p.H) * 2u + ch * 16u) = o;
            if (k == 0u) cx.sm_phase(kSmFirstCombined);
            cx.sm_phase(kSmCombineDone);
        }
    }

    // ---- exit: an aborted SM lets the loader's copies in flight land (a bounded wait on the barriers of the stages it
    //      issued last) before the shared memory goes away
    if (warp == 0 && cx.aborted()) {
        const uint32_t issued = *reinterpret_cast<volatile uint32_t*>(&c.issued), nst = tiles ? p.nstage_wide : static_cast<uint32_t>(p.nstage);
        #pragma unroll 1
        for (uint32_t k = issued > nst ? issued - nst : 0u; k < issued; ++k) {
            const uint32_t s = k % nst, ph = (k / nst) & 1u;
            for (uint32_t spin = 0; spin < 400000u && !mbar_try_wait(&c.full[s], ph); ++spin) { }
        }
        if (tiles) {                                       // likewise the token records (and the last tile header) still on their way
            const uint32_t rissued = *reinterpret_cast<volatile uint32_t*>(&c.rissued), nr = p.nrec;
            #pragma unroll 1
            for (uint32_t k = rissued > nr ? rissued - nr : 0u; k < rissued; ++k) {
                const uint32_t s = k % nr, ph = (k / nr) & 1u;
                for (uint32_t spin = 0; spin < 400000u && !mbar_try_wait(&c.rfull[s], ph); ++spin) { }
            }
            for (uint32_t spin = 0; spin < 2000u; ++spin) __nanosleep(100);      // (a 512 B header copy: microseconds at most)
        }
    }
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(c.tmem_base, kTmemCols); }
    if (tid == 0) {
        if (bid == 0) cx.stamp(kStampExit);
        cx.stamp_max(kStampLastExit, globaltimer_ns());
        cx.sm_phase(kSmExit);
    }
}

}  // namespace mm
