/* C ABI of the B200 (sm_100a) expert-parallel MegaMoE layer.
 *
 * Plain pointers and sizes only; every function returns an `mm_status` code and never throws.
 * The library is what a host binding (ctypes, pybind, cgo ...) loads in place of the reference's
 * `deep_gemm._C` mega-MoE entry points. File:line citations name the reference interface that
 * each entry point replaces (paths relative to the reference project's root).
 */
#ifndef MEGAMOE_B200_H_
#define MEGAMOE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum mm_status {
    MM_OK = 0,
    MM_ERR_INVALID_ARGUMENT = 1,   /* shape / pointer check failed (reference: DG_HOST_ASSERT -> RuntimeError) */
    MM_ERR_UNSUPPORTED = 2,        /* a limit of this build (hidden size, experts per rank, ...) */
    MM_ERR_CUDA = 3,               /* a CUDA runtime call failed; see mm_last_cuda_error() */
    MM_ERR_DEVICE_TIMEOUT = 4,     /* a bounded device-side wait expired; see mm_read_device_status() */
    MM_ERR_DEVICE_CAPACITY = 5     /* a device-side table overflowed (rows received / tasks per SM) */
};

enum mm_act_format { MM_FMT_MXFP4 = 0, MM_FMT_NVFP4 = 1, MM_FMT_FP8 = 2 };
enum mm_engine { MM_ENGINE_UMMA = 0 /* tcgen05 block-scaled MMA */, MM_ENGINE_CHECK = 1 /* same kernel, CUDA-core dot products: on-device cross-check */ };

/* Static description of one layer instance; identical on every rank except `rank`. */
typedef struct mm_config {
    int32_t num_ranks;                 /* expert-parallel group size, 1..8 */
    int32_t rank;
    int32_t num_experts;               /* global; num_experts / num_ranks experts live on each rank (<= 64) */
    int32_t num_max_tokens_per_rank;
    int32_t num_topk;
    int32_t hidden;                    /* multiple of 512, <= 4096 */
    int32_t intermediate;              /* multiple of 256 */
    int32_t act_format;                /* enum mm_act_format */
    int32_t num_sms;                   /* persistent grid size; 0 = all SMs of the current device */
} mm_config_t;

/* Byte offsets of the regions inside one rank's symmetric buffer.
 * Replaces `get_symm_buffer_size_for_mega_moe` + its slicing lambda (sm100_b200/apis_mega.hpp:23-171). */
typedef struct mm_layout {
    int64_t total_bytes;
    int64_t off_ctrl;          /* per-SM launch counters, device status words, phase stamps, per-SM time records */
    int64_t off_x;             /* [T_max][x_row_bytes]   quantised tokens (caller or frontend writes) */
    int64_t off_x_sf;          /* [T_max][x_sf_row_bytes] one scale byte per `vec` elements, K-major */
    int64_t off_topk_idx;      /* [T_max][topk] int64, -1 = masked slot */
    int64_t off_topk_weights;  /* [T_max][topk] float */
    int64_t off_rx;            /* [2 parities][num_ranks sources][rx_region_bytes] receive pool: a 32 B header line (row count), then
                                  rx_cap_rows rows of 2 * rx_row_bytes; every 8 bytes = {4 data bytes, launch flag} */
    int64_t off_mid;           /* [mid_rows][2 * mid_row_bytes] requantised SwiGLU output (local), flagged 8-byte words */
    int64_t off_mid_sf;        /* [mid_rows][intermediate / 64] flagged words {scale bytes of 64 columns, launch flag} */
    int64_t off_comb;          /* [T_max][topk][hidden] bf16 expert outputs written back by the peers, as flagged 8-byte words
                                  {2 bf16, launch flag}: 4 bytes per element */
    int64_t off_red;           /* [256 SMs][2 phases][2][16][128] float partial sums of weight tiles split between SMs (local) */
    int64_t off_cnt;           /* [2 phases][cnt_per_phase] uint32 contributors that have parked their part of a tile (local) */
    int64_t off_logits;        /* [min(T_max, 256)][num_experts] 16 B records {half logit, launch flag} x 2 of the fused router frontend */
    int64_t x_row_bytes, x_sf_row_bytes;
    int64_t rx_row_bytes, rx_cap_rows;
    int64_t mid_rows, mid_row_bytes, mid_sf_row_bytes;
    int64_t cnt_per_phase;
    int32_t sf_vec;            /* elements per scale byte of the activation format */
    int32_t ctrl_bytes;        /* bytes of the control block at off_ctrl */
    int64_t rx_region_bytes;   /* bytes of one (parity, source) region of the receive pool */
    /* Launches with more than 16 received rows: rows sorted by expert into ready-made 16-token operand tiles (local). */
    int64_t off_token_tiles;   /* [tile_capacity][token_tile_bytes] received rows of one token tile (16 or 32 rows) of one expert: 32 row
                                  records of 16 B {source rank, token, slot, weight}, then per streamed K unit the unit's 128 B of every
                                  row in the tensor core's shared-memory order (128 B swizzle) and the unit's scale-word slots */
    int64_t off_mid_tiles;     /* [tile_capacity][mid_tile_bytes] the same, without the row records, for the requantised SwiGLU output */
    int64_t off_arrive;        /* [2 parities][2][tile_capacity] uint32: rows of a token tile written / L1 weight tiles of a mid tile written */
    int64_t tile_capacity, token_tile_bytes, mid_tile_bytes;
} mm_layout_t;

/* Geometry of the pre-tiled weight stream produced by the load-time transform.
 * Replaces the layout contract of `transform_weights_for_mega_moe` (sm100_b200/mega___init__.py:81-111). */
typedef struct mm_weight_geometry {
    int32_t tile_rows;         /* 128 weight rows per tile */
    int32_t unit_k;            /* K elements per streamed unit */
    int32_t unit_weight_bytes; /* swizzled weight bytes of one unit */
    int32_t unit_sf_bytes;     /* scale planes of one unit */
    int32_t unit_bytes;        /* stride between units */
    int32_t sf_vec;            /* elements per weight scale byte */
} mm_weight_geometry_t;

typedef struct mm_launch_args {
    void* buffer;                    /* this rank's symmetric buffer (mm_layout.total_bytes) */
    void* const* peer_buffers;       /* num_ranks device pointers, peer_buffers[rank] == buffer */
    const void* l1_weights;          /* pre-tiled stream [E_local][2I/128][H/unit_k][unit_bytes] */
    const void* l2_weights;          /* pre-tiled stream [E_local][H/128][I/unit_k][unit_bytes] */
    void* y;                         /* bf16 [num_tokens][hidden], caller-owned */
    int32_t num_tokens;              /* tokens of this rank in this call (rows of y) */
    int32_t engine;                  /* enum mm_engine */
    int32_t* cumulative_local_expert_recv_stats;   /* optional int32 [E_local], += rows received */
    float activation_clamp;          /* < 0 or inf: no clamp */
    int32_t fast_math;               /* 1: __expf + approximate reciprocal in the SwiGLU */
    float x_global_scale, l1_global_scale, l2_global_scale, mid_global_scale;   /* NVFP4 per-tensor scales; 1.0 otherwise */
    float timeout_ms;                /* budget of every device-side wait; <= 0: 2000 ms */
    const void* input_region;        /* optional: where the kernel reads this call's x / x_sf / topk_idx / topk_weights from,
                                        laid out like the buffer's bytes [off_x, off_rx). NULL: the buffer's own views. A
                                        pinned (device-mapped) host mirror here lets one launch replace copy + launch. */
} mm_launch_args_t;

/* Router frontend: bf16 router GEMM, top-k selection, token quantisation into the buffer views.
 * Replaces `launch_router_quant_topk_frontend` (sm100_b200/fe_sm100/fable_frontend.h:48-52). */
typedef struct mm_frontend_args {
    const void* hidden_states;       /* bf16 [num_tokens][hidden] */
    const void* router_weight;       /* bf16 [num_experts][hidden] */
    const float* expert_bias;        /* optional float [num_experts] (score_mode 1) */
    int32_t num_tokens;
    int32_t score_mode;              /* 0: softmax over the selected logits; 1: sigmoid + bias selection, renormalised */
    void* workspace;                 /* mm_frontend_workspace_bytes() bytes of device memory (partial logits of the two-kernel frontend;
                                        the single-kernel path keeps its own inside the buffer and only requires it non-NULL) */
    float x_global_scale;
} mm_frontend_args_t;

/* sm100_b200/apis_mega.hpp:23-171 (buffer sizing) */
int mm_get_layout(const mm_config_t* cfg, mm_layout_t* out);
/* sm100_b200/mega___init__.py:81-111 (weight layout contract) */
int mm_get_weight_geometry(int32_t act_format, mm_weight_geometry_t* out);
/* Load-time weight transform as one CUDA copy kernel: `transform_weights_for_mega_moe` (sm100_b200/mega___init__.py:81-111:
 * gate/up interleave of L1, 4 x 32 transposition of the scale words) fused with the scale-layout step the reference runs
 * before it (`transform_sf_into_required_layout`, csrc/apis/layout.hpp:14-60: int32 MN-major scale words, or fp32 scales
 * that are first turned into UE8M0 / E4M3 bytes). w_packed: E2M1 pairs [groups][n][k/2]; sf: int32 words (4 scale bytes of
 * consecutive K blocks each) or fp32 scales, addressed as sf[g * stride_e + row * stride_n + i * stride_k] in elements of
 * its type; out_stream: [groups][n/128][k/256][mm_weight_geometry.unit_bytes]. */
int mm_transform_weights(const void* w_packed, const void* sf, int32_t sf_is_fp32, int64_t sf_stride_e, int64_t sf_stride_n,
                         int64_t sf_stride_k, int32_t num_groups, int32_t n, int32_t k, int32_t sf_vec, int32_t interleave_gate_up,
                         void* out_stream, void* stream);
/* Row-wise cast to packed E2M1 with one fp32 scale per gran_k elements, the arithmetic of `per_token_cast_to_fp4`
 * (deep_gemm/utils/math.py:85-111). x: bf16 or fp32 [m][k]; packed_out [m][k/2]; sf_out fp32 [m][k/gran_k]. */
/* Largest magnitude of a bf16 or fp32 tensor of n elements (16-byte aligned), written as one float to device memory: the
 * calibration step of an NVFP4 per-tensor global scale, `absmax / (6 * 448)` (the rule of the benchmark's NVFP4
 * configuration; the reference's SM100 operator has no global-scale argument and its tests compute none). */
int mm_tensor_absmax(const void* x, int32_t x_is_bf16, int64_t n, float* absmax_out, void* stream);
int mm_cast_rows_to_fp4(const void* x, int32_t x_is_bf16, int32_t m, int32_t k, int32_t gran_k, int32_t use_ue8m0,
                        void* packed_out, float* sf_out, void* stream);
/* sm100_b200/apis_mega.hpp:544-552 (`get_token_alignment_for_mega_moe`) */
int32_t mm_get_token_alignment(void);
/* sm100_b200/apis_mega.hpp:173-358 (`fp8_fp4_mega_moe`, `fp4_fp4_mega_moe`): asynchronous launch on `stream` */
int mm_mega_moe_launch(const mm_config_t* cfg, const mm_launch_args_t* args, void* stream);
/* sm100_b200/fe_sm100/fable_frontend.h:48-52 (`launch_router_quant_topk_frontend`) */
int mm_frontend_launch(const mm_config_t* cfg, void* buffer, const mm_frontend_args_t* args, void* stream);
/* sm100_b200/fe_sm100/fe_binding.cpp:8-35 (`fe_workspace_bytes`) */
int64_t mm_frontend_workspace_bytes(const mm_config_t* cfg);
/* sm100_b200/fe_sm100/fe_binding.cpp:8-35 (`fe_forward`) over `launch_router_quant_topk_frontend`
 * (sm100_b200/fe_sm100/fable_frontend.h:48-52), with the reference's argument list: bf16 hidden [m][h], bf16 router
 * weight [e][h] -> quantised rows x [m][h/2] (mode 3 MXFP4, 4 NVFP4) or [m][h] (mode 2 FP8), scale bytes x_sf
 * [m][h/32] (h/16 for NVFP4), topk_idx int64 [m][topk], topk_weights float [m][topk]; softmax over the selected
 * logits, an all-zero row is left unrouted (idx -1, weight 0). m <= 64, topk = 8. `l2_persist` is accepted and ignored. */
int mm_fe_forward(const void* hidden, const void* router_weight, void* x, void* x_sf, void* topk_idx, void* topk_weights,
                  void* workspace, int64_t workspace_bytes, int32_t m, int32_t h, int32_t e, int32_t topk, int32_t mode,
                  int32_t l2_persist, void* stream);
/* sm100_b200/fe_sm100/fe_binding.cpp:30 (`fe_workspace_bytes(e)`): 256 + 4 * 64 * e * 4 */
int64_t mm_fe_workspace_bytes(int32_t e);
/* sm100_b200/fe_sm100/fe_binding.cpp:31 (`fe_router_ctas(m, h, e, topk)`): CTAs of the router-logits kernel */
int32_t mm_fe_router_ctas(int32_t m, int32_t h, int32_t e, int32_t topk);
/* Router frontend and layer as ONE persistent kernel (the frontend's outputs still land in the buffer views). */
int mm_mega_moe_from_hidden_launch(const mm_config_t* cfg, const mm_launch_args_t* args,
                                   const mm_frontend_args_t* fe, void* stream);
/* The symmetric window without torch: every rank allocates its buffer (device memory, zeroed) and gets a handle of
 * MM_WINDOW_HANDLE_BYTES that it publishes to the other ranks of the node by whatever the host has (the Python mirror
 * all-gathers them over its NCCL group); with all handles, mm_window_open maps the peers' buffers and returns the table
 * of base pointers mm_launch_args.peer_buffers wants. One-time set-up; nothing of it runs per layer. Replaces
 * `symm_mem.empty` + `symm_mem.rendezvous` (sm100_b200/mega___init__.py:43-47). mm_window_close unmaps the peers and
 * frees the own buffer (pass NULL to keep it). */
#define MM_WINDOW_HANDLE_BYTES 64
int mm_window_alloc(int64_t bytes, void** ptr_out, uint8_t handle_out[MM_WINDOW_HANDLE_BYTES]);
int mm_window_open(const uint8_t* handles, int32_t num_ranks, int32_t rank, void* own_ptr, void** peer_ptrs_out);
int mm_window_close(void* const* peer_ptrs, int32_t num_ranks, int32_t rank, void* own_ptr_to_free);
/* Zero the control block and every flagged region: the launch numbering restarts (after an aborted launch or at
 * creation). The reference's only remedy is re-creating the buffer (sm100_b200/mega___init__.py:43-47). Callers synchronise the ranks around it. */
int mm_reset(const mm_config_t* cfg, void* buffer, void* stream);
/* Synchronises `stream`, then copies the 16 device status words: [0] first failure (0 = none; code | sm << 8 |
 * detail << 16), [1] launches seen, [2] rows per token tile (16 or 32) when the latest launch kept its rows as tile images (more than
 * 16 received rows), else 0, [3..] diagnostics. The reference traps instead (sm100_b200/layout_mega_moe.cuh:13-19). */
int mm_read_device_status(const mm_config_t* cfg, const void* buffer, uint32_t out_words[16], void* stream);
/* Synchronises `stream`, then copies the 32 phase stamps (globaltimer ns) of the last launch. Slots, SM 0 unless
 * noted: 0 first instruction, 1 dispatched, 2 header lines of all ranks seen, 3 scheduled, 4 tasks done, 5 prologue
 * done, 7 exit, 8 last SM out, 9 fused frontend done, 10 last SM's tasks done, 11 last SM scheduled, 12 first
 * instruction of the earliest SM, 13 first weight request (L2 prefetch or shared-memory copy) of any SM, 14 last
 * streamed weight unit found in shared memory by any SM (8, 10, 11, 14: maxima over the SMs; 12, 13: minima).
 * Replaces the `DG_SM100_PHASE_STAMPS_PTR` facility (sm100_b200/sm100_fp4_fp4_mega_moe.cuh:97-128). */
int mm_read_phase_stamps(const mm_config_t* cfg, const void* buffer, uint64_t out_stamps[32], void* stream);
/* Synchronises `stream`, then copies the per-SM phase times of the last launch: out[sm * 32 + slot], globaltimer ns,
 * 0 = not reached. Slots: 0 first instruction, 1 prologue done, 2 own rows listed, 3 row counts known, 4 scheduled,
 * 5 first weight copy issued, 6 first weight unit landed, 7 first task's tokens staged, 8 first task's MMAs done,
 * 9 first epilogue done, 10 last L1 epilogue done, 11 first L2 task's rows staged, 12 tasks done, 13 first combine
 * item written, 14 last combine item written, 15 exit, 16..30 when the SM's weight units 0..14 were found landed, 31 latest copy of a received row into the row cache. The reference's per-CTA frontend stamps are the model
 * (sm100_b200/fe_sm100/fable_frontend_device.cuh:46-54). */
int mm_read_sm_phases(const mm_config_t* cfg, const void* buffer, uint64_t* out_256x32, void* stream);
/* Development knobs, process-wide, read at every launch. The reference reads its own from DG_SM100_* environment
 * variables (sm100_b200/sm100_fp4_fp4_mega_moe.hpp:215-248). MM_TUNE_KNOBS is a bit mask: 1 the spare warp asks for a
 * live expert's weights (L2 prefetch) as soon as it learns of the expert, 2 every SM lists the rows of this rank's own
 * tokens from topk_idx instead of waiting for the own-rank header line, 4 warps start the combine when their role ends,
 * 8 the token-staging warps rehearse their code on made-up tasks while the dispatch is in flight, 16 launches with more
 * than 16 received rows sort them into ready-made operand tiles in global memory and fetch a task's tokens by bulk copies. */
enum mm_tuning_key { MM_TUNE_KNOBS = 0, MM_TUNE_STAGES = 1 /* ring depth, 0 = default */,
                     MM_TUNE_PREFETCH_W1_EXPERTS = 2, MM_TUNE_PREFETCH_W2_EXPERTS = 3 /* experts prefetched per launch at most */,
                     MM_TUNE_ROW_CACHE = 4 /* 1: received rows are fetched into shared memory before the weight stream starts */,
                     MM_TUNE_COUNT = 5 };
int mm_set_tuning(int32_t key, int32_t value);
int32_t mm_get_tuning(int32_t key);

/* Bytes of the library's built-in working memory (one array per GPU, resident from library load to process exit). */
#define MM_STATIC_SCRATCH_BYTES (16ll * 1024 * 1024)

typedef struct mm_static_args {
    const void* x;                   /* packed tokens [num_tokens][hidden / 2] (device) */
    const void* x_sf;                /* scale bytes [num_tokens][hidden / vec] (device) */
    const int64_t* topk_idx;         /* [num_tokens][topk], -1 = masked slot (device) */
    const float* topk_weights;       /* [num_tokens][topk] (device) */
    const void* l1_weights;          /* pre-tiled streams, as in mm_launch_args */
    const void* l2_weights;
    void* y;                         /* bf16 [num_tokens][hidden] (device) */
    int32_t num_tokens;
    int32_t fast_math;
    int32_t* cumulative_local_expert_recv_stats;   /* optional */
    float activation_clamp;
    float x_global_scale, l1_global_scale, l2_global_scale, mid_global_scale;
    float timeout_ms;
    uint32_t* device_status_out;     /* optional: 16 words (device), filled on the stream after the kernel */
} mm_static_args_t;

/* No counterpart in the reference. A single-rank launch of the layer for hosts that must not allocate device
 * memory at call time: serving processes that carve up the GPU once at start-up and forbid cudaMalloc afterwards
 * (it synchronises the device and can fail late), plugins running inside another framework's memory plan, real-time
 * loops. The caller passes only inputs, weights and the output; the layer's working memory (receive pool,
 * intermediate rows, combine rows, counters) is the library's own fixed array of MM_STATIC_SCRATCH_BYTES per GPU.
 * The call issues memsets, device-to-device copies of the inputs and the kernel on `stream`, and calls no cudaMalloc,
 * cudaFree or other allocating routine. Limits: num_ranks must be 1; a configuration whose mm_layout.total_bytes
 * exceeds MM_STATIC_SCRATCH_BYTES is refused with MM_ERR_UNSUPPORTED (mm_last_cuda_error() says by how much).
 * The first call on each device looks up the array's device address, and the first launch of a format on a device may
 * load the kernel's module and sets its shared-memory attribute; make that call outside any stream capture.
 * All calls on a GPU share the one array and it keeps the previous call's bytes (the call clears the parts that must
 * start from zero), so two calls that overlap on the GPU, e.g. on different streams, race: serialise them. */
int mm_mega_moe_launch_static_scratch(const mm_config_t* cfg, const mm_static_args_t* args, void* stream);
const char* mm_status_string(int status);
const char* mm_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif  /* MEGAMOE_B200_H_ */
