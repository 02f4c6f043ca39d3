"""B200-native (sm_100a) expert-parallel MegaMoE layer behind the reference's operator surface."""
from .mega import (SymmBuffer, get_symm_buffer_for_mega_moe, get_token_alignment_for_mega_moe,
                   transform_weights_for_mega_moe, fp4_fp4_mega_moe, fp8_fp4_mega_moe, fe_forward, fe_forward_into_buffer, fe_router_ctas, fe_workspace_bytes,
                   mega_moe_from_hidden, set_tuning, nvfp4_global_scale)
from . import quant

__all__ = ['SymmBuffer', 'get_symm_buffer_for_mega_moe', 'get_token_alignment_for_mega_moe',
           'transform_weights_for_mega_moe', 'fp4_fp4_mega_moe', 'fp8_fp4_mega_moe', 'fe_forward', 'fe_forward_into_buffer', 'fe_router_ctas',
           'fe_workspace_bytes', 'mega_moe_from_hidden', 'set_tuning', 'nvfp4_global_scale', 'quant']
