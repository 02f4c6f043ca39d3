"""ctypes binding of the C ABI declared in include/megamoe_b200.h. There is no fallback: a missing library is an error."""
import ctypes
import os

from .build import CHECK_LIB_PATH, LIB_PATH

MM_OK = 0
FMT = {'mxfp4': 0, 'nvfp4': 1, 'fp8': 2}
ENGINE = {'umma': 0, 'check': 1}


class MMConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        'num_ranks', 'rank', 'num_experts', 'num_max_tokens_per_rank', 'num_topk', 'hidden', 'intermediate',
        'act_format', 'num_sms')]


class MMLayout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in (
        'total_bytes', 'off_ctrl', 'off_x', 'off_x_sf', 'off_topk_idx', 'off_topk_weights', 'off_rx',
        'off_mid', 'off_mid_sf', 'off_comb', 'off_red', 'off_cnt', 'off_logits', 'x_row_bytes', 'x_sf_row_bytes', 'rx_row_bytes', 'rx_cap_rows',
        'mid_rows', 'mid_row_bytes', 'mid_sf_row_bytes', 'cnt_per_phase')] + [('sf_vec', ctypes.c_int32), ('ctrl_bytes', ctypes.c_int32),
                                                   ('rx_region_bytes', ctypes.c_int64)] + [(n, ctypes.c_int64) for n in (
        'off_token_tiles', 'off_mid_tiles', 'off_arrive', 'tile_capacity', 'token_tile_bytes', 'mid_tile_bytes')]


class MMWeightGeometry(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        'tile_rows', 'unit_k', 'unit_weight_bytes', 'unit_sf_bytes', 'unit_bytes', 'sf_vec')]


class MMLaunchArgs(ctypes.Structure):
    _fields_ = [
        ('buffer', ctypes.c_void_p), ('peer_buffers', ctypes.POINTER(ctypes.c_void_p)),
        ('l1_weights', ctypes.c_void_p), ('l2_weights', ctypes.c_void_p), ('y', ctypes.c_void_p),
        ('num_tokens', ctypes.c_int32), ('engine', ctypes.c_int32),
        ('cumulative_local_expert_recv_stats', ctypes.c_void_p),
        ('activation_clamp', ctypes.c_float), ('fast_math', ctypes.c_int32),
        ('x_global_scale', ctypes.c_float), ('l1_global_scale', ctypes.c_float),
        ('l2_global_scale', ctypes.c_float), ('mid_global_scale', ctypes.c_float),
        ('timeout_ms', ctypes.c_float), ('input_region', ctypes.c_void_p)]


class MMFrontendArgs(ctypes.Structure):
    _fields_ = [
        ('hidden_states', ctypes.c_void_p), ('router_weight', ctypes.c_void_p), ('expert_bias', ctypes.c_void_p),
        ('num_tokens', ctypes.c_int32), ('score_mode', ctypes.c_int32), ('workspace', ctypes.c_void_p),
        ('x_global_scale', ctypes.c_float)]


class MMStaticArgs(ctypes.Structure):
    _fields_ = [
        ('x', ctypes.c_void_p), ('x_sf', ctypes.c_void_p), ('topk_idx', ctypes.c_void_p), ('topk_weights', ctypes.c_void_p),
        ('l1_weights', ctypes.c_void_p), ('l2_weights', ctypes.c_void_p), ('y', ctypes.c_void_p),
        ('num_tokens', ctypes.c_int32), ('fast_math', ctypes.c_int32),
        ('cumulative_local_expert_recv_stats', ctypes.c_void_p), ('activation_clamp', ctypes.c_float),
        ('x_global_scale', ctypes.c_float), ('l1_global_scale', ctypes.c_float),
        ('l2_global_scale', ctypes.c_float), ('mid_global_scale', ctypes.c_float),
        ('timeout_ms', ctypes.c_float), ('device_status_out', ctypes.c_void_p)]


STATIC_SCRATCH_BYTES = 16 * 1024 * 1024
TUNE = {'knobs': 0, 'stages': 1, 'prefetch_w1_experts': 2, 'prefetch_w2_experts': 3, 'row_cache': 4}
KNOB_PREFETCH, KNOB_OWN_ROWS, KNOB_EARLY_COMBINE = 1, 2, 4
WINDOW_HANDLE_BYTES = 64

EXPORTS = ('mm_get_layout', 'mm_get_weight_geometry', 'mm_get_token_alignment', 'mm_mega_moe_launch',
           'mm_frontend_launch', 'mm_frontend_workspace_bytes', 'mm_mega_moe_from_hidden_launch', 'mm_reset',
           'mm_read_device_status', 'mm_read_phase_stamps', 'mm_status_string', 'mm_last_cuda_error',
           'mm_mega_moe_launch_static_scratch', 'mm_set_tuning', 'mm_get_tuning', 'mm_read_sm_phases', 'mm_fe_forward', 'mm_fe_workspace_bytes', 'mm_fe_router_ctas', 'mm_transform_weights', 'mm_cast_rows_to_fp4', 'mm_tensor_absmax', 'mm_window_alloc', 'mm_window_open', 'mm_window_close')

_libs = {}


def load(check: bool = False) -> ctypes.CDLL:
    """Load the compiled library; raises if it has not been built (`python -m <package>.build`). `check=True` loads the
    test build that also carries the CUDA-core cross-check engine."""
    if check in _libs:
        return _libs[check]
    path = CHECK_LIB_PATH if check else LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(f'{path} is missing: build it with `python -m hopper_megamoe_basedondeepgemm_b200.build` '
                           '(nvcc, sm_100a). There is no CPU or eager fallback for this operator.')
    lib = ctypes.CDLL(path)
    P = ctypes.POINTER
    lib.mm_get_layout.argtypes = [P(MMConfig), P(MMLayout)]
    lib.mm_get_weight_geometry.argtypes = [ctypes.c_int32, P(MMWeightGeometry)]
    lib.mm_get_token_alignment.restype = ctypes.c_int32
    lib.mm_mega_moe_launch.argtypes = [P(MMConfig), P(MMLaunchArgs), ctypes.c_void_p]
    lib.mm_frontend_launch.argtypes = [P(MMConfig), ctypes.c_void_p, P(MMFrontendArgs), ctypes.c_void_p]
    lib.mm_frontend_workspace_bytes.argtypes = [P(MMConfig)]
    lib.mm_frontend_workspace_bytes.restype = ctypes.c_int64
    lib.mm_mega_moe_from_hidden_launch.argtypes = [P(MMConfig), P(MMLaunchArgs), P(MMFrontendArgs), ctypes.c_void_p]
    lib.mm_mega_moe_launch_static_scratch.argtypes = [P(MMConfig), P(MMStaticArgs), ctypes.c_void_p]
    lib.mm_set_tuning.argtypes = [ctypes.c_int32, ctypes.c_int32]
    lib.mm_get_tuning.argtypes = [ctypes.c_int32]
    lib.mm_get_tuning.restype = ctypes.c_int32
    lib.mm_reset.argtypes = [P(MMConfig), ctypes.c_void_p, ctypes.c_void_p]
    lib.mm_read_device_status.argtypes = [P(MMConfig), ctypes.c_void_p, P(ctypes.c_uint32), ctypes.c_void_p]
    lib.mm_read_phase_stamps.argtypes = [P(MMConfig), ctypes.c_void_p, P(ctypes.c_uint64), ctypes.c_void_p]
    lib.mm_read_sm_phases.argtypes = [P(MMConfig), ctypes.c_void_p, P(ctypes.c_uint64), ctypes.c_void_p]
    lib.mm_fe_forward.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64] + [ctypes.c_int32] * 6 + [ctypes.c_void_p]
    lib.mm_fe_workspace_bytes.argtypes = [ctypes.c_int32]
    lib.mm_fe_workspace_bytes.restype = ctypes.c_int64
    lib.mm_fe_router_ctas.argtypes = [ctypes.c_int32] * 4
    lib.mm_fe_router_ctas.restype = ctypes.c_int32
    lib.mm_transform_weights.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_int64] + [ctypes.c_int32] * 5 + [ctypes.c_void_p, ctypes.c_void_p]
    lib.mm_tensor_absmax.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.mm_cast_rows_to_fp4.argtypes = [ctypes.c_void_p] + [ctypes.c_int32] * 5 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.mm_window_alloc.argtypes = [ctypes.c_int64, P(ctypes.c_void_p), ctypes.c_char_p]
    lib.mm_window_open.argtypes = [ctypes.c_char_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, P(ctypes.c_void_p)]
    lib.mm_window_close.argtypes = [P(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.mm_status_string.argtypes = [ctypes.c_int]
    lib.mm_status_string.restype = ctypes.c_char_p
    lib.mm_last_cuda_error.restype = ctypes.c_char_p
    _libs[check] = lib
    return lib


def check(status: int, what: str) -> None:
    """Status code -> RuntimeError, like the reference's DG_HOST_ASSERT -> RuntimeError path."""
    if status != MM_OK:
        lib = load()
        msg = lib.mm_status_string(status).decode()
        extra = lib.mm_last_cuda_error().decode() if status == 3 else ''
        raise RuntimeError(f'{what}: {msg}{(" (" + extra + ")") if extra else ""}')
