// C ABI of the library: argument checks, buffer layout, launch parameters. No torch types, no exceptions.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <cstdlib>

#include "../../include/megamoe_b200.h"
#include "mm_kernel.cuh"
#include "mm_frontend.cuh"
#include "mm_prep.cuh"

namespace {

thread_local char g_cuda_error[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", what, cudaGetErrorString(e));
    return MM_ERR_CUDA;
}
#define MM_CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return cuda_fail(e_, #call); } while (0)

inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

int sf_vec_of(int fmt) { return fmt == MM_FMT_NVFP4 ? 16 : 32; }

// development knobs (mm_set_tuning): kernel feature bits, ring depth (0 = chosen from the shared-memory plan), and how
// many experts' W1 / W2 the scout may prefetch into the L2 in one launch
// (the L2 prefetch of live experts' weights is off by default: measured, it does not shorten the weight stream - bulk
// copies from the L2 are barely faster than from HBM here - and its traffic delays the launch's small critical loads)
int g_tuning[MM_TUNE_COUNT] = {mm::kKnobOwnRows | mm::kKnobEarlyCombine | mm::kKnobTileImages, 0, 14, 14, 1};

int check_config(const mm_config_t* c) {
    if (c == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (c->num_ranks < 1 || c->num_ranks > mm::kMaxRanks || c->rank < 0 || c->rank >= c->num_ranks) return MM_ERR_INVALID_ARGUMENT;
    if (c->num_experts <= 0 || c->num_experts % c->num_ranks != 0) return MM_ERR_INVALID_ARGUMENT;
    if (c->num_experts / c->num_ranks > mm::kMaxLocalExperts) return MM_ERR_UNSUPPORTED;
    if (c->num_topk < 1 || c->num_topk > 32 || c->num_max_tokens_per_rank < 1 || c->num_max_tokens_per_rank > 32768) return MM_ERR_INVALID_ARGUMENT;
    if (c->hidden <= 0 || c->hidden % 512 != 0 || c->hidden > 4096) return MM_ERR_UNSUPPORTED;
    if (c->intermediate <= 0 || c->intermediate % 256 != 0 || c->intermediate > 4096) return MM_ERR_UNSUPPORTED;
    if (c->act_format != MM_FMT_MXFP4 && c->act_format != MM_FMT_NVFP4 && c->act_format != MM_FMT_FP8) return MM_ERR_UNSUPPORTED;
    return MM_OK;
}

int grid_size(const mm_config_t* cfg, int* out) {
    int g = cfg->num_sms;
    if (g <= 0) {
        int dev = 0;
        MM_CUDA(cudaGetDevice(&dev));
        MM_CUDA(cudaDeviceGetAttribute(&g, cudaDevAttrMultiProcessorCount, dev));
    }
    if (g > 256 || g < cfg->num_ranks) return MM_ERR_UNSUPPORTED;
    *out = g;
    return MM_OK;
}

}  // namespace

extern "C" {

const char* mm_status_string(int s) {
    switch (s) {
        case MM_OK: return "ok";
        case MM_ERR_INVALID_ARGUMENT: return "invalid argument";
        case MM_ERR_UNSUPPORTED: return "unsupported configuration";
        case MM_ERR_CUDA: return "CUDA runtime error";
        case MM_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case MM_ERR_DEVICE_CAPACITY: return "device-side table capacity exceeded";
        default: return "unknown status";
    }
}

const char* mm_last_cuda_error(void) { return g_cuda_error; }

int32_t mm_get_token_alignment(void) { return 16; }

int mm_set_tuning(int32_t key, int32_t value) {
    if (key < 0 || key >= MM_TUNE_COUNT || value < 0) return MM_ERR_INVALID_ARGUMENT;
    g_tuning[key] = value;
    return MM_OK;
}

int32_t mm_get_tuning(int32_t key) { return key >= 0 && key < MM_TUNE_COUNT ? g_tuning[key] : -1; }

int mm_get_weight_geometry(int32_t act_format, mm_weight_geometry_t* out) {
    if (out == nullptr || (act_format != MM_FMT_MXFP4 && act_format != MM_FMT_NVFP4 && act_format != MM_FMT_FP8)) return MM_ERR_INVALID_ARGUMENT;
    const int vec = sf_vec_of(act_format);
    out->tile_rows = mm::kTileRows;
    out->unit_k = mm::kUnitK;
    out->unit_weight_bytes = mm::kUnitWBytes;
    out->unit_sf_bytes = (mm::kUnitK / (4 * vec)) * 512;
    out->unit_bytes = out->unit_weight_bytes + out->unit_sf_bytes;
    out->sf_vec = vec;
    return MM_OK;
}

int mm_get_layout(const mm_config_t* c, mm_layout_t* out) {
    const int st = check_config(c);
    if (st != MM_OK) return st;
    if (out == nullptr) return MM_ERR_INVALID_ARGUMENT;
    memset(out, 0, sizeof(*out));
    const int vec = sf_vec_of(c->act_format);
    const int64_t e_local = c->num_experts / c->num_ranks;
    const int64_t t_max = c->num_max_tokens_per_rank;
    out->sf_vec = vec;
    const bool a8 = c->act_format == MM_FMT_FP8;           // E4M3 tokens: one byte per element, UE8M0 scale per 32
    out->x_row_bytes = a8 ? c->hidden : c->hidden / 2;
    out->x_sf_row_bytes = c->hidden / vec;
    out->rx_row_bytes = out->x_row_bytes + out->x_sf_row_bytes + 16;
    out->rx_cap_rows = t_max * (c->num_topk < e_local ? c->num_topk : e_local);
    out->mid_rows = out->rx_cap_rows * c->num_ranks + mm::kTileTokens * e_local;
    out->mid_row_bytes = a8 ? c->intermediate : c->intermediate / 2;
    out->mid_sf_row_bytes = align_up(c->intermediate / vec, 16);
    int64_t off = 0;
    auto take = [&](int64_t bytes) { const int64_t o = off; off = align_up(off + bytes, 1024); return o; };
    out->off_ctrl = take(mm::kCtrlBytes);
    out->ctrl_bytes = mm::kCtrlBytes;
    out->off_x = take(t_max * out->x_row_bytes);
    out->off_x_sf = take(t_max * out->x_sf_row_bytes);
    out->off_topk_idx = take(t_max * c->num_topk * 8);
    out->off_topk_weights = take(t_max * c->num_topk * 4);
    out->rx_region_bytes = align_up(32 + out->rx_cap_rows * 2 * out->rx_row_bytes, 128);
    out->off_rx = take(2 * c->num_ranks * out->rx_region_bytes);
    out->off_mid = take(out->mid_rows * 2 * out->mid_row_bytes);                 // flagged words: twice the payload
    out->off_mid_sf = take(out->mid_rows * (c->intermediate / 64) * 8);         // one flagged word per (row, L1 tile)
    out->off_comb = take(t_max * c->num_topk * c->hidden * 4);
    const int64_t n_max = (2 * c->intermediate > c->hidden ? 2 * c->intermediate : c->hidden) / mm::kTileRows;
    out->cnt_per_phase = (out->mid_rows / mm::kTileTokens) * n_max;
    out->off_red = take(256 /* SMs */ * 2 /* phases */ * 2 /* slots */ * mm::kTileTokens * mm::kTileRows * 4);
    out->off_cnt = take(2 * out->cnt_per_phase * 4);
    // partial router logits of the fused frontend: 16 B per (token, expert), flagged with the launch number
    out->off_logits = take((t_max < mm::kFeMaxFusedTokens ? t_max : mm::kFeMaxFusedTokens) * c->num_experts * 16);
    // tile images of the launches with more than 16 received rows: token bytes of 16 rows, then one 16 B slot per (scale word, row)
    out->tile_capacity = out->mid_rows / mm::kTileTokens;
    {
        // per tile: 32 row records of 16 B (token tiles only), then per streamed K unit a record of up to 32 rows x 128 B
        // and the unit's scale-word slots (16 B per (scale word, row))
        const int64_t rec32 = mm::kWideTokens * 128 + (mm::kUnitK / (4 * vec)) * mm::kWideTokens * 16;
        out->token_tile_bytes = mm::kWideTokens * 16 + (c->hidden / mm::kUnitK) * rec32;
        out->mid_tile_bytes = (c->intermediate / mm::kUnitK) * rec32;
    }
    out->off_token_tiles = take(out->tile_capacity * out->token_tile_bytes);
    out->off_mid_tiles = take(out->tile_capacity * out->mid_tile_bytes);
    out->off_arrive = take(2 * 2 * out->tile_capacity * 4);
    out->total_bytes = off;
    return MM_OK;
}

// ----------------------------------------------------------------------------- symmetric window without torch
int mm_window_alloc(int64_t bytes, void** ptr_out, uint8_t handle_out[MM_WINDOW_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) <= MM_WINDOW_HANDLE_BYTES, "handle size");
    if (bytes <= 0 || ptr_out == nullptr || handle_out == nullptr) return MM_ERR_INVALID_ARGUMENT;
    void* p = nullptr;
    MM_CUDA(cudaMalloc(&p, static_cast<size_t>(bytes)));
    cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "mm_window_alloc"); }
    memset(handle_out, 0, MM_WINDOW_HANDLE_BYTES);
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return MM_OK;
}

int mm_window_open(const uint8_t* handles, int32_t num_ranks, int32_t rank, void* own_ptr, void** peer_ptrs_out) {
    if (handles == nullptr || peer_ptrs_out == nullptr || own_ptr == nullptr || num_ranks < 1 || num_ranks > mm::kMaxRanks ||
        rank < 0 || rank >= num_ranks) return MM_ERR_INVALID_ARGUMENT;
    for (int r = 0; r < num_ranks; ++r) peer_ptrs_out[r] = nullptr;
    for (int r = 0; r < num_ranks; ++r) {
        if (r == rank) { peer_ptrs_out[r] = own_ptr; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + static_cast<size_t>(r) * MM_WINDOW_HANDLE_BYTES, sizeof(h));
        const cudaError_t e = cudaIpcOpenMemHandle(&peer_ptrs_out[r], h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q) if (q != rank && peer_ptrs_out[q] != nullptr) cudaIpcCloseMemHandle(peer_ptrs_out[q]);
            return cuda_fail(e, "mm_window_open");
        }
    }
    return MM_OK;
}

int mm_window_close(void* const* peer_ptrs, int32_t num_ranks, int32_t rank, void* own_ptr_to_free) {
    if (peer_ptrs != nullptr)
        for (int r = 0; r < num_ranks; ++r)
            if (r != rank && peer_ptrs[r] != nullptr) MM_CUDA(cudaIpcCloseMemHandle(peer_ptrs[r]));
    if (own_ptr_to_free != nullptr) MM_CUDA(cudaFree(own_ptr_to_free));
    return MM_OK;
}

int mm_reset(const mm_config_t* cfg, void* buffer, void* stream) {
    mm_layout_t L;
    const int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (buffer == nullptr) return MM_ERR_INVALID_ARGUMENT;
    // the launch counters restart from zero, so every flagged word of earlier launches must go too: the receive pool,
    // the intermediate pool and the combine buffer are cleared with the control block and the split-tile counters
    MM_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(buffer) + L.off_ctrl, 0, L.off_x - L.off_ctrl, static_cast<cudaStream_t>(stream)));
    MM_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(buffer) + L.off_rx, 0, L.total_bytes - L.off_rx, static_cast<cudaStream_t>(stream)));
    return MM_OK;
}

int mm_read_device_status(const mm_config_t* cfg, const void* buffer, uint32_t out_words[16], void* stream) {
    mm_layout_t L;
    const int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (buffer == nullptr || out_words == nullptr) return MM_ERR_INVALID_ARGUMENT;
    MM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    MM_CUDA(cudaMemcpy(out_words, static_cast<const uint8_t*>(buffer) + L.off_ctrl + mm::kCtrlStatus, 64, cudaMemcpyDeviceToHost));
    const uint32_t code = out_words[0] & 0xFFu;
    if (code == 0) return MM_OK;
    return (code == mm::kErrMetaCapacity || code == mm::kErrTaskCapacity) ? MM_ERR_DEVICE_CAPACITY : MM_ERR_DEVICE_TIMEOUT;
}

int mm_read_phase_stamps(const mm_config_t* cfg, const void* buffer, uint64_t out_stamps[32], void* stream) {
    mm_layout_t L;
    const int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (buffer == nullptr || out_stamps == nullptr) return MM_ERR_INVALID_ARGUMENT;
    MM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    MM_CUDA(cudaMemcpy(out_stamps, static_cast<const uint8_t*>(buffer) + L.off_ctrl + mm::kCtrlStamps, 256, cudaMemcpyDeviceToHost));
    // per-SM records -> slot 12 (first instruction of the earliest SM) and slot 13 (first weight request of any SM)
    static thread_local uint64_t per_sm[512];
    MM_CUDA(cudaMemcpy(per_sm, static_cast<const uint8_t*>(buffer) + L.off_ctrl + mm::kCtrlSmEntry, sizeof(per_sm), cudaMemcpyDeviceToHost));
    uint64_t first_in = ~0ull, first_w = ~0ull;
    for (int i = 0; i < 256; ++i) {
        if (per_sm[i] != 0 && per_sm[i] < first_in) first_in = per_sm[i];
        if (per_sm[256 + i] != 0 && per_sm[256 + i] < first_w) first_w = per_sm[256 + i];
    }
    out_stamps[12] = first_in == ~0ull ? 0 : first_in;
    out_stamps[13] = first_w == ~0ull ? 0 : first_w;
    return MM_OK;
}

}  // extern "C"

static int fill_params(const mm_config_t* cfg, const mm_launch_args_t* a, mm::KParams* P, int* grid, size_t* smem_bytes) {
    mm_layout_t L;
    int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (a == nullptr || a->buffer == nullptr || a->peer_buffers == nullptr || a->l1_weights == nullptr || a->l2_weights == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (a->num_tokens < 0 || a->num_tokens > cfg->num_max_tokens_per_rank) return MM_ERR_INVALID_ARGUMENT;
    if (a->num_tokens > 0 && a->y == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (a->peer_buffers[cfg->rank] != a->buffer) return MM_ERR_INVALID_ARGUMENT;
    st = grid_size(cfg, grid);
    if (st != MM_OK) return st;
    mm_weight_geometry_t wg;
    mm_get_weight_geometry(cfg->act_format, &wg);
    mm::KParams& p = *P;
    memset(&p, 0, sizeof(p));
    p.R = cfg->num_ranks; p.rank = cfg->rank; p.e_local = cfg->num_experts / cfg->num_ranks; p.topk = cfg->num_topk;
    p.H = cfg->hidden; p.I = cfg->intermediate; p.T = a->num_tokens; p.cap = static_cast<int>(L.rx_cap_rows);
    p.n1_tiles = 2 * p.I / mm::kTileRows; p.n2_tiles = p.H / mm::kTileRows;
    p.k1_units = p.H / mm::kUnitK; p.k2_units = p.I / mm::kUnitK;
    if (p.n1_tiles > 255 || p.n2_tiles > 255) return MM_ERR_UNSUPPORTED;
    p.unit_bytes = wg.unit_bytes;
    p.x_row_bytes = static_cast<int>(L.x_row_bytes); p.x_sf_row_bytes = static_cast<int>(L.x_sf_row_bytes);
    p.rx_row_bytes = static_cast<int>(L.rx_row_bytes); p.rx_region = L.rx_region_bytes;
    p.mid_row_bytes = static_cast<int>(L.mid_row_bytes); p.mid_sf_row_bytes = static_cast<int>(L.mid_sf_row_bytes);
    p.has_clamp = (a->activation_clamp >= 0.f && std::isfinite(a->activation_clamp)) ? 1 : 0;
    p.clamp = a->activation_clamp; p.fast_math = a->fast_math;
    const float xg = a->x_global_scale > 0.f ? a->x_global_scale : 1.f, g1 = a->l1_global_scale > 0.f ? a->l1_global_scale : 1.f;
    const float g2 = a->l2_global_scale > 0.f ? a->l2_global_scale : 1.f, gm = a->mid_global_scale > 0.f ? a->mid_global_scale : 1.f;
    p.l1_scale = xg * g1; p.l2_scale = g2 * gm; p.mid_gs = gm;
    for (int r = 0; r < p.R; ++r) {
        if (a->peer_buffers[r] == nullptr) return MM_ERR_INVALID_ARGUMENT;
        p.peer[r] = static_cast<uint8_t*>(a->peer_buffers[r]);
    }
    p.w1 = static_cast<const uint8_t*>(a->l1_weights); p.w2 = static_cast<const uint8_t*>(a->l2_weights);
    p.y = static_cast<__nv_bfloat16*>(a->y); p.stats = a->cumulative_local_expert_recv_stats;
    p.off_ctrl = L.off_ctrl; p.off_x = L.off_x; p.off_x_sf = L.off_x_sf;
    p.inp = a->input_region != nullptr ? static_cast<const uint8_t*>(a->input_region) - L.off_x : static_cast<const uint8_t*>(a->buffer);
    p.knobs = static_cast<uint32_t>(g_tuning[MM_TUNE_KNOBS]);
    p.pf_w1_max = static_cast<uint32_t>(g_tuning[MM_TUNE_PREFETCH_W1_EXPERTS]);
    p.pf_w2_max = static_cast<uint32_t>(g_tuning[MM_TUNE_PREFETCH_W2_EXPERTS]);
    p.off_topk_idx = L.off_topk_idx; p.off_topk_w = L.off_topk_weights; p.off_rx = L.off_rx;
    p.off_mid = L.off_mid; p.off_mid_sf = L.off_mid_sf; p.off_comb = L.off_comb;
    p.off_red = L.off_red; p.off_cnt = L.off_cnt; p.cnt_per_phase = static_cast<int>(L.cnt_per_phase);
    p.off_token_tiles = L.off_token_tiles; p.off_mid_tiles = L.off_mid_tiles; p.off_arrive = L.off_arrive;
    p.tile_capacity = static_cast<uint32_t>(L.tile_capacity);
    p.token_tile_bytes = static_cast<uint32_t>(L.token_tile_bytes); p.mid_tile_bytes = static_cast<uint32_t>(L.mid_tile_bytes);
    const double tmo = a->timeout_ms > 0.f ? a->timeout_ms : 2000.0;
    p.timeout_ns = static_cast<unsigned long long>(tmo * 1e6);
    // shared memory plan: [stages][token tiles][token scale chunks][output tile][accumulator tile][widened units (FP8)]
    const int kmax = p.H > p.I ? p.H : p.I;
    const int vec = sf_vec_of(cfg->act_format);
    const bool a8 = cfg->act_format == MM_FMT_FP8;
    p.act_bytes = a8 ? mm::kTileTokens * kmax : mm::kTileTokens * kmax / 2;
    p.asf_bytes = static_cast<uint32_t>(align_up(kmax / vec, 16) / 4 * 256);     // 256 B per scale word of the K axis
    const size_t xbytes = a8 ? 2 * mm::kXbufBytes : 0;
    const size_t budget = 232448 - sizeof(mm::Ctl) - 1024 /* alignment slack */ - 768;
    // two token staging buffers when that leaves at least four stream stages, else one
    // (with one, the kernel still runs two 8-row halves when no expert has more than 8 rows: two scale-slot areas always)
    p.nab = 2;
    // output tile and accumulator tile: sized for 32-row token tiles, which only the formats with tile images use
    const size_t otile_bytes = a8 ? mm::kOtileBytes / 2 : mm::kOtileBytes, vt_bytes = a8 ? mm::kVtBytes / 2 : mm::kVtBytes;
    size_t fixed = p.nab * p.act_bytes + 2 * p.asf_bytes + otile_bytes + vt_bytes + xbytes;
    if (fixed + 4 * static_cast<size_t>(p.unit_bytes) > budget) {
        p.nab = 1;
        fixed = p.nab * p.act_bytes + 2 * p.asf_bytes + otile_bytes + vt_bytes + xbytes;
    }
    if (fixed + 2 * static_cast<size_t>(p.unit_bytes) > budget) return MM_ERR_UNSUPPORTED;
    int nstage = static_cast<int>((budget - fixed) / p.unit_bytes);
    // A short ring is faster than a deep one: the loader runs ahead into the next phase's weights, and with many stages
    // that prefetch competes with the stream the current phase is waiting for (measured: 4 stages beat 8 by 2 us).
    const int want = g_tuning[MM_TUNE_STAGES] > 0 ? g_tuning[MM_TUNE_STAGES] : mm::kDefaultStages;
    if (nstage > want) nstage = want;
    if (nstage > mm::kMaxStages) nstage = mm::kMaxStages;
    // FP8 activations: the two widening warp groups take the units alternately, and a group must see every use of a
    // stage it waits on (a group that skipped a stage's previous use could take its barrier's older phase for the one it
    // wants): with an even ring depth a stage always belongs to the same group
    if (a8) nstage &= ~1;
    if (nstage < 2) return MM_ERR_UNSUPPORTED;
    p.nstage = nstage;
    // dispatching SMs per destination: one per ~8 expected rows (one row per copying warp), at most G / R
    {
        int nd = (p.T * p.topk) / (p.R * 8);
        if (nd > *grid / p.R) nd = *grid / p.R;
        p.ndisp = nd < 1 ? 1 : nd;
    }
    // launches that work from tile images use the stages and the token staging area as one longer weight ring, and the
    // token region as a ring of token records (32 rows x 128 B + scale-word slots per slot)
    p.wide_stage_bytes = p.unit_bytes;
    p.rec_slot_bytes = mm::kWideTokens * 128 + (mm::kUnitK / (4 * vec)) * mm::kWideTokens * 16;
    p.sm_act = nstage * p.unit_bytes;
    p.sm_asf = p.sm_act + p.nab * p.act_bytes;
    p.sm_otile = p.sm_asf + 2 * p.asf_bytes;
    p.stage_region = p.sm_otile - p.sm_act;
    p.nstage_wide = a8 ? 0u : p.sm_otile / p.wide_stage_bytes;
    if (p.nstage_wide > 6u) p.nstage_wide = 6u;
    p.sm_vt = p.sm_otile + static_cast<uint32_t>(otile_bytes);
    p.sm_xbuf = static_cast<uint32_t>(align_up(p.sm_vt + vt_bytes, 1024));
    size_t used = a8 ? p.sm_xbuf + xbytes : p.sm_vt + vt_bytes;
    // token region: the first 16 received rows (tokens + scale bytes) are fetched into what the plan leaves free, either as
    // one swizzled token tile with its scale slots (launches with at most 16 received rows) or as a plain row cache
    p.rc_row_bytes = static_cast<uint32_t>(L.x_row_bytes + L.x_sf_row_bytes);
    p.sm_rcache = static_cast<uint32_t>(align_up(used, 1024));
    p.rc_rows = 0;
    {
        const size_t as_cache = 16ull * p.rc_row_bytes, as_tile = static_cast<size_t>(p.act_bytes) + p.asf_bytes;
        const size_t region = as_cache > as_tile ? as_cache : as_tile;
        if (g_tuning[MM_TUNE_ROW_CACHE] != 0 && !a8 && p.sm_rcache + region + 1024 + 256 <= 232448 - sizeof(mm::Ctl) - 768) {
            p.rc_rows = 16;
            // launches with tile images keep their ring of token records here: as many slots as fit, eight at most
            const size_t room = 232448 - sizeof(mm::Ctl) - 768 - 1024 - 256 - p.sm_rcache;
            p.sm_rec = p.sm_rcache;
            p.nrec = static_cast<uint32_t>(room / p.rec_slot_bytes);
            if (p.nrec > mm::kMaxRecSlots) p.nrec = mm::kMaxRecSlots;
            const size_t rec_region = static_cast<size_t>(p.nrec) * p.rec_slot_bytes;
            used = p.sm_rcache + (region > rec_region ? region : rec_region);
        }
    }
    *smem_bytes = used + 1024 + 256;
    if (static_cast<size_t>(p.T) * p.topk * 4 > p.stage_region) return MM_ERR_UNSUPPORTED;
    return MM_OK;
}

static bool wants_tile_images(const mm::KParams& p) {
    return (p.knobs & mm::kKnobTileImages) != 0u && p.nstage_wide >= 3u && p.nrec >= 2u && static_cast<long long>(p.T) * p.topk > mm::kTileTokens;
}

template <int kVec, bool kUmma, bool kFe = false, bool kA8 = false, bool kTiles = false>
static int launch_variant(const mm::KParams& p, int grid, size_t smem_bytes, cudaStream_t stream) {
    auto kern = mm::mega_moe_kernel<kVec, kUmma, kFe, kA8, kTiles>;
    // the opt-in shared-memory size is a per-device function attribute: set once per (variant, device), raised on demand
    static int attr_bytes[64] = {};
    int dev = 0;
    MM_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || attr_bytes[dev] < static_cast<int>(smem_bytes)) {
        MM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)));
        if (dev >= 0 && dev < 64) attr_bytes[dev] = static_cast<int>(smem_bytes);
    }
    kern<<<grid, kA8 ? mm::kThreads + mm::kNumExpThreads : mm::kThreads, smem_bytes, stream>>>(p);
    MM_CUDA(cudaGetLastError());
    return MM_OK;
}

extern "C" {

int mm_mega_moe_launch(const mm_config_t* cfg, const mm_launch_args_t* a, void* stream) {
    mm::KParams p;
    int grid = 0;
    size_t smem_bytes = 0;
    const int st = fill_params(cfg, a, &p, &grid, &smem_bytes);
    if (st != MM_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool umma = a->engine == MM_ENGINE_UMMA;
    if (cfg->act_format == MM_FMT_FP8)                                     // tensor-core engine only
        return umma ? launch_variant<32, true, false, true>(p, grid, smem_bytes, s) : MM_ERR_UNSUPPORTED;
#ifdef MM_WITH_CHECK_ENGINE
    // the CUDA-core cross-check engine is test infrastructure: only the test build of the library carries it
    if (!umma)
        return cfg->act_format == MM_FMT_MXFP4 ? launch_variant<32, false>(p, grid, smem_bytes, s) : launch_variant<16, false>(p, grid, smem_bytes, s);
#else
    if (!umma) return MM_ERR_UNSUPPORTED;
#endif
    // Two builds of the tensor-core kernel for the 4-bit activation formats: one that can work from tile images (launches
    // with more than 16 received rows) and one without that code, whose start-up path is shorter. Either is correct for
    // any input; a rank with at most 16 routed rows of its own takes the lean one (the decode-size launches).
    if (wants_tile_images(p))
        return cfg->act_format == MM_FMT_MXFP4 ? launch_variant<32, true, false, false, true>(p, grid, smem_bytes, s)
                                               : launch_variant<16, true, false, false, true>(p, grid, smem_bytes, s);
    return cfg->act_format == MM_FMT_MXFP4 ? launch_variant<32, true>(p, grid, smem_bytes, s) : launch_variant<16, true>(p, grid, smem_bytes, s);
}

int mm_read_sm_phases(const mm_config_t* cfg, const void* buffer, uint64_t* out, void* stream) {
    mm_layout_t L;
    const int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (buffer == nullptr || out == nullptr) return MM_ERR_INVALID_ARGUMENT;
    MM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    MM_CUDA(cudaMemcpy(out, static_cast<const uint8_t*>(buffer) + L.off_ctrl + mm::kCtrlSmPhase, 256 * mm::kSmPhaseSlots * 8, cudaMemcpyDeviceToHost));
    return MM_OK;
}

int64_t mm_frontend_workspace_bytes(const mm_config_t* cfg) {
    if (cfg == nullptr) return -1;
    return static_cast<int64_t>(cfg->num_max_tokens_per_rank) * cfg->num_experts * 16 + 256;
}

int mm_frontend_launch(const mm_config_t* cfg, void* buffer, const mm_frontend_args_t* fe, void* stream) {
    mm_layout_t L;
    int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (buffer == nullptr || fe == nullptr || fe->hidden_states == nullptr || fe->router_weight == nullptr || fe->workspace == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (fe->num_tokens < 0 || fe->num_tokens > cfg->num_max_tokens_per_rank) return MM_ERR_INVALID_ARGUMENT;
    if (cfg->num_topk != 8 || cfg->num_experts > 1024) return MM_ERR_UNSUPPORTED;
    if (cfg->num_experts < cfg->num_topk) return MM_ERR_INVALID_ARGUMENT;      // fewer experts than routes per token
    if (fe->score_mode == 1 && fe->expert_bias == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (fe->num_tokens == 0) return MM_OK;
    int grid = 0;
    st = grid_size(cfg, &grid);
    if (st != MM_OK) return st;
    mm::FeParams q;
    memset(&q, 0, sizeof(q));
    q.hidden = static_cast<const __nv_bfloat16*>(fe->hidden_states);
    q.router_w = static_cast<const __nv_bfloat16*>(fe->router_weight);
    q.bias = fe->expert_bias;
    q.logits = reinterpret_cast<float*>(static_cast<uint8_t*>(fe->workspace) + 256);
    q.arrive = reinterpret_cast<uint32_t*>(fe->workspace);
    q.T = fe->num_tokens; q.H = cfg->hidden; q.E = cfg->num_experts; q.topk = cfg->num_topk;
    q.score_mode = fe->score_mode; q.fmt = cfg->act_format;
    q.x_gs = fe->x_global_scale > 0.f ? fe->x_global_scale : 1.f;
    uint8_t* b = static_cast<uint8_t*>(buffer);
    q.x = b + L.off_x; q.x_sf = b + L.off_x_sf;
    q.topk_idx = reinterpret_cast<long long*>(b + L.off_topk_idx);
    q.topk_w = reinterpret_cast<float*>(b + L.off_topk_weights);
    q.x_row_bytes = static_cast<int>(L.x_row_bytes); q.x_sf_row_bytes = static_cast<int>(L.x_sf_row_bytes);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    mm::frontend_logits_kernel<<<grid, 256, 0, s>>>(q);
    MM_CUDA(cudaGetLastError());
    const int sel_blocks = (q.T + 3) / 4;
    mm::frontend_select_quant_kernel<<<sel_blocks, 128, q.E * 2 * 4 * 4, s>>>(q);
    MM_CUDA(cudaGetLastError());
    return MM_OK;
}

int mm_transform_weights(const void* w_packed, const void* sf, int32_t sf_is_fp32, int64_t sf_stride_e, int64_t sf_stride_n,
                         int64_t sf_stride_k, int32_t num_groups, int32_t n, int32_t k, int32_t sf_vec, int32_t interleave_gate_up,
                         void* out_stream, void* stream) {
    if (w_packed == nullptr || sf == nullptr || out_stream == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (num_groups <= 0 || n <= 0 || k <= 0 || n % 128 != 0 || k % 256 != 0) return MM_ERR_INVALID_ARGUMENT;
    if (sf_vec != 16 && sf_vec != 32) return MM_ERR_UNSUPPORTED;
    if (interleave_gate_up && n % 16 != 0) return MM_ERR_INVALID_ARGUMENT;
    mm::PrepParams q;
    memset(&q, 0, sizeof(q));
    q.w = static_cast<const uint8_t*>(w_packed); q.sf = sf;
    q.sf_stride_e = sf_stride_e; q.sf_stride_n = sf_stride_n; q.sf_stride_k = sf_stride_k;
    q.sf_is_fp32 = sf_is_fp32; q.E = num_groups; q.N = n; q.K = k; q.vec = sf_vec; q.interleave = interleave_gate_up;
    q.out = static_cast<uint8_t*>(out_stream);
    q.planes = mm::kUnitK / (4 * sf_vec);
    q.unit_bytes = mm::kUnitWBytes + q.planes * 512;
    const long long units = static_cast<long long>(num_groups) * (n / 128) * (k / 256);
    if (units > 0x7FFFFFFFll) return MM_ERR_UNSUPPORTED;
    mm::pretile_weights_kernel<<<static_cast<unsigned>(units), 256, 0, static_cast<cudaStream_t>(stream)>>>(q);
    MM_CUDA(cudaGetLastError());
    return MM_OK;
}

int mm_cast_rows_to_fp4(const void* x, int32_t x_is_bf16, int32_t m, int32_t k, int32_t gran_k, int32_t use_ue8m0,
                        void* packed_out, float* sf_out, void* stream) {
    if (x == nullptr || packed_out == nullptr || sf_out == nullptr || m < 0 || k <= 0) return MM_ERR_INVALID_ARGUMENT;
    if ((gran_k != 16 && gran_k != 32 && gran_k != 64 && gran_k != 128) || k % gran_k != 0) return MM_ERR_UNSUPPORTED;
    if (m == 0) return MM_OK;
    const long long threads = static_cast<long long>(m) * (k / 8);
    const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (x_is_bf16)
        mm::cast_rows_fp4_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), m, k, gran_k, use_ue8m0,
                                                                      static_cast<uint8_t*>(packed_out), sf_out);
    else
        mm::cast_rows_fp4_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), m, k, gran_k, use_ue8m0,
                                                              static_cast<uint8_t*>(packed_out), sf_out);
    MM_CUDA(cudaGetLastError());
    return MM_OK;
}

int mm_tensor_absmax(const void* x, int32_t x_is_bf16, int64_t n, float* absmax_out, void* stream) {
    if (x == nullptr || absmax_out == nullptr || n < 0) return MM_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0u) return MM_ERR_INVALID_ARGUMENT;      // 16 B loads
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MM_CUDA(cudaMemsetAsync(absmax_out, 0, sizeof(float), s));
    if (n == 0) return MM_OK;
    const long long per = x_is_bf16 ? 8 : 4;
    long long blocks = (n / per + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 1184 ? 1184 : blocks);                               // eight blocks per SM at most
    if (x_is_bf16)
        mm::absmax_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, reinterpret_cast<uint32_t*>(absmax_out));
    else
        mm::absmax_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const float*>(x), n, reinterpret_cast<uint32_t*>(absmax_out));
    MM_CUDA(cudaGetLastError());
    return MM_OK;
}

int64_t mm_fe_workspace_bytes(int32_t e) { return e > 0 ? 256 + static_cast<int64_t>(4) * 64 * e * 4 : -1; }

int32_t mm_fe_router_ctas(int32_t m, int32_t h, int32_t e, int32_t topk) {
    (void)m; (void)h; (void)e; (void)topk;
    int dev = 0, g = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return g;                              // the logits kernel runs one CTA per SM whatever the shape
}

int mm_fe_forward(const void* hidden, const void* router_weight, void* x, void* x_sf, void* topk_idx, void* topk_weights,
                  void* workspace, int64_t workspace_bytes, int32_t m, int32_t h, int32_t e, int32_t topk, int32_t mode,
                  int32_t l2_persist, void* stream) {
    (void)l2_persist;                      // accepted for the reference's argument list; the router matrix is read once per launch
    if (hidden == nullptr || router_weight == nullptr || x == nullptr || x_sf == nullptr || topk_idx == nullptr ||
        topk_weights == nullptr || workspace == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (m < 1 || m > 64 || h <= 0 || h % 256 != 0 || h > 4096) return MM_ERR_INVALID_ARGUMENT;
    if (topk != 8 || e > 1024) return MM_ERR_UNSUPPORTED;
    if (e < topk) return MM_ERR_INVALID_ARGUMENT;
    if (mode < 2 || mode > 4) return MM_ERR_UNSUPPORTED;          // 2 FP8 / 3 MXFP4 / 4 NVFP4 (0 and 1 are Hopper formats)
    if (workspace_bytes < 256 + static_cast<int64_t>(m) * e * 16) return MM_ERR_INVALID_ARGUMENT;
    int dev = 0, grid = 0;
    MM_CUDA(cudaGetDevice(&dev));
    MM_CUDA(cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev));
    const int fmt = mode == 2 ? MM_FMT_FP8 : (mode == 3 ? MM_FMT_MXFP4 : MM_FMT_NVFP4);
    mm::FeParams q;
    memset(&q, 0, sizeof(q));
    q.hidden = static_cast<const __nv_bfloat16*>(hidden);
    q.router_w = static_cast<const __nv_bfloat16*>(router_weight);
    q.logits = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    q.arrive = reinterpret_cast<uint32_t*>(workspace);
    q.T = m; q.H = h; q.E = e; q.topk = topk; q.score_mode = 0; q.fmt = fmt; q.x_gs = 1.f;
    q.x = static_cast<uint8_t*>(x); q.x_sf = static_cast<uint8_t*>(x_sf);
    q.topk_idx = static_cast<long long*>(topk_idx); q.topk_w = static_cast<float*>(topk_weights);
    q.x_row_bytes = fmt == MM_FMT_FP8 ? h : h / 2;
    q.x_sf_row_bytes = h / sf_vec_of(fmt);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    mm::frontend_logits_kernel<<<grid, 256, 0, s>>>(q);
    MM_CUDA(cudaGetLastError());
    mm::frontend_select_quant_kernel<<<(m + 3) / 4, 128, q.E * 2 * 4 * 4, s>>>(q);
    MM_CUDA(cudaGetLastError());
    return MM_OK;
}

int mm_mega_moe_from_hidden_launch(const mm_config_t* cfg, const mm_launch_args_t* a, const mm_frontend_args_t* fe, void* stream) {
    mm::KParams p;
    int grid = 0;
    size_t smem_bytes = 0;
    int st = fill_params(cfg, a, &p, &grid, &smem_bytes);
    if (st != MM_OK) return st;
    if (fe == nullptr || (fe->hidden_states == nullptr && fe->num_tokens > 0) || fe->router_weight == nullptr || fe->workspace == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (fe->num_tokens != a->num_tokens) return MM_ERR_INVALID_ARGUMENT;
    if (cfg->num_topk != 8 || cfg->num_experts > 1024) return MM_ERR_UNSUPPORTED;
    if (cfg->num_experts < cfg->num_topk) return MM_ERR_INVALID_ARGUMENT;      // fewer experts than routes per token
    if (fe->score_mode == 1 && fe->expert_bias == nullptr) return MM_ERR_INVALID_ARGUMENT;
    const bool a8 = cfg->act_format == MM_FMT_FP8;
    if (static_cast<size_t>(cfg->num_experts) * 2 * 4 * ((mm::kThreads + (a8 ? mm::kNumExpThreads : 0)) / 32) > p.stage_region) return MM_ERR_UNSUPPORTED;
    if (fe->num_tokens > mm::kFeMaxFusedTokens) return MM_ERR_UNSUPPORTED;
    mm_layout_t L;
    mm_get_layout(cfg, &L);
    uint8_t* b = static_cast<uint8_t*>(a->buffer);
    mm::FeParams& q = p.fe;
    q.hidden = static_cast<const __nv_bfloat16*>(fe->hidden_states);
    q.router_w = static_cast<const __nv_bfloat16*>(fe->router_weight);
    q.bias = fe->expert_bias;
    q.logits = reinterpret_cast<float*>(b + L.off_logits);       // inside the buffer: `mm_reset` clears the flagged records with it
    q.arrive = nullptr;
    q.T = fe->num_tokens; q.H = cfg->hidden; q.E = cfg->num_experts; q.topk = cfg->num_topk;
    q.score_mode = fe->score_mode; q.fmt = cfg->act_format;
    q.x_gs = fe->x_global_scale > 0.f ? fe->x_global_scale : 1.f;
    q.x = b + L.off_x; q.x_sf = b + L.off_x_sf;
    q.topk_idx = reinterpret_cast<long long*>(b + L.off_topk_idx);
    q.topk_w = reinterpret_cast<float*>(b + L.off_topk_weights);
    q.x_row_bytes = static_cast<int>(L.x_row_bytes); q.x_sf_row_bytes = static_cast<int>(L.x_sf_row_bytes);
    p.fe_enabled = 1;
    // (the dispatching SMs also select the routes, each of them for all tokens: `fill_params` chose one SM per eight rows)
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a->engine != MM_ENGINE_UMMA) return MM_ERR_UNSUPPORTED;     // the cross-check engine takes pre-routed inputs only
    if (a8) return fe->num_tokens == 0 ? launch_variant<32, true, false, true>(p, grid, smem_bytes, s)
                                       : launch_variant<32, true, true, true>(p, grid, smem_bytes, s);
    if (fe->num_tokens == 0) return cfg->act_format == MM_FMT_MXFP4 ? launch_variant<32, true>(p, grid, smem_bytes, s)
                                                                    : launch_variant<16, true>(p, grid, smem_bytes, s);
    if (wants_tile_images(p))
        return cfg->act_format == MM_FMT_MXFP4 ? launch_variant<32, true, true, false, true>(p, grid, smem_bytes, s)
                                               : launch_variant<16, true, true, false, true>(p, grid, smem_bytes, s);
    return cfg->act_format == MM_FMT_MXFP4 ? launch_variant<32, true, true>(p, grid, smem_bytes, s)
                                           : launch_variant<16, true, true>(p, grid, smem_bytes, s);
}

// ----------------------------------------------------------------------------- launch without any allocation
// Working memory of mm_mega_moe_launch_static_scratch: one fixed array per GPU that loads this library, held until
// the process exits. In host code the symbol below is only a handle; the device address comes from
// cudaGetSymbolAddress (looked up once per device, with that device current) and that address is what the kernel gets.
static __device__ __align__(256) unsigned char g_static_scratch[MM_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
unsigned char* g_static_scratch_addr[kMaxDevices] = {};
}  // namespace

int mm_mega_moe_launch_static_scratch(const mm_config_t* cfg, const mm_static_args_t* a, void* stream) {
    if (cfg == nullptr || a == nullptr) return MM_ERR_INVALID_ARGUMENT;
    if (cfg->num_ranks != 1 || cfg->rank != 0) {
        snprintf(g_cuda_error, sizeof(g_cuda_error), "static scratch serves one rank only: peers cannot map it");
        return MM_ERR_UNSUPPORTED;
    }
    mm_layout_t L;
    int st = mm_get_layout(cfg, &L);
    if (st != MM_OK) return st;
    if (L.total_bytes > static_cast<int64_t>(MM_STATIC_SCRATCH_BYTES)) {
        snprintf(g_cuda_error, sizeof(g_cuda_error), "configuration needs %lld bytes of working memory, the static scratch holds %lld",
                 static_cast<long long>(L.total_bytes), static_cast<long long>(MM_STATIC_SCRATCH_BYTES));
        return MM_ERR_UNSUPPORTED;
    }
    if (a->num_tokens < 0 || a->num_tokens > cfg->num_max_tokens_per_rank) return MM_ERR_INVALID_ARGUMENT;
    if (a->num_tokens > 0 && (a->x == nullptr || a->x_sf == nullptr || a->topk_idx == nullptr || a->topk_weights == nullptr || a->y == nullptr))
        return MM_ERR_INVALID_ARGUMENT;
    int dev = 0;
    MM_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return MM_ERR_UNSUPPORTED;
    if (g_static_scratch_addr[dev] == nullptr) {
        // first call on this device: resolve the array's device address (do this before any stream capture)
        void* ptr = nullptr;
        MM_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_static_scratch_addr[dev] = static_cast<unsigned char*>(ptr);
    }
    unsigned char* scratch = g_static_scratch_addr[dev];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps the previous call's contents: the control block, the arrival flags and the split-tile counters
    // must start from zero (the launch counters restart with them, so every call runs as the buffer's first launch),
    // and with the counters every flagged word of the receive pool and the combine buffer
    // (the split-tile partial sums between them are always written before they are read: not cleared)
    MM_CUDA(cudaMemsetAsync(scratch + L.off_ctrl, 0, L.off_x - L.off_ctrl, s));
    MM_CUDA(cudaMemsetAsync(scratch + L.off_rx, 0, L.off_red - L.off_rx, s));
    MM_CUDA(cudaMemsetAsync(scratch + L.off_cnt, 0, L.off_token_tiles - L.off_cnt, s));
    MM_CUDA(cudaMemsetAsync(scratch + L.off_arrive, 0, L.total_bytes - L.off_arrive, s));      // (the tile images need no clearing)
    const size_t t = static_cast<size_t>(a->num_tokens);
    if (t > 0) {
        MM_CUDA(cudaMemcpyAsync(scratch + L.off_x, a->x, t * L.x_row_bytes, cudaMemcpyDeviceToDevice, s));
        MM_CUDA(cudaMemcpyAsync(scratch + L.off_x_sf, a->x_sf, t * L.x_sf_row_bytes, cudaMemcpyDeviceToDevice, s));
        MM_CUDA(cudaMemcpyAsync(scratch + L.off_topk_idx, a->topk_idx, t * cfg->num_topk * 8, cudaMemcpyDeviceToDevice, s));
        MM_CUDA(cudaMemcpyAsync(scratch + L.off_topk_weights, a->topk_weights, t * cfg->num_topk * 4, cudaMemcpyDeviceToDevice, s));
    }
    void* peers[1] = {scratch};
    mm_launch_args_t la;
    memset(&la, 0, sizeof(la));
    la.buffer = scratch; la.peer_buffers = peers;
    la.l1_weights = a->l1_weights; la.l2_weights = a->l2_weights; la.y = a->y; la.num_tokens = a->num_tokens;
    la.engine = MM_ENGINE_UMMA; la.cumulative_local_expert_recv_stats = a->cumulative_local_expert_recv_stats;
    la.activation_clamp = a->activation_clamp; la.fast_math = a->fast_math;
    la.x_global_scale = a->x_global_scale; la.l1_global_scale = a->l1_global_scale;
    la.l2_global_scale = a->l2_global_scale; la.mid_global_scale = a->mid_global_scale; la.timeout_ms = a->timeout_ms;
    st = mm_mega_moe_launch(cfg, &la, stream);
    if (st != MM_OK) return st;
    if (a->device_status_out != nullptr)
        MM_CUDA(cudaMemcpyAsync(a->device_status_out, scratch + L.off_ctrl + mm::kCtrlStatus, 64, cudaMemcpyDeviceToDevice, s));
    return MM_OK;
}

}  // extern "C"
