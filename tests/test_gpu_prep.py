"""Load-time preparation kernels on the GPU: the pre-tiled weight stream byte for byte against its torch restatement, the
row-wise E2M1 cast bit for bit against the vectors generated from the reference's `per_token_cast_to_fp4`."""
import ctypes
import os

import numpy as np
import pytest
import torch

import hopper_megamoe_basedondeepgemm_b200 as mm
from hopper_megamoe_basedondeepgemm_b200 import _lib, quant

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def _weights(fmt, e, n, k, seed):
    g = torch.Generator(device='cuda').manual_seed(seed)
    w = (torch.randn((e, n, k), generator=g, device='cuda') * 0.05).to(torch.bfloat16)
    return quant.cast_grouped_weights_to_fp4(w, fmt)            # (packed int8 [E, N, K/2], int32 words MN-major)


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4'])
@pytest.mark.parametrize('interleave', [False, True])
def test_transform_kernel_equals_the_torch_restatement(fmt, interleave):
    vec = quant.SF_VEC[fmt]
    q, sf = _weights(fmt, 3, 512, 1024, 7)
    want = quant.pretile_weights(quant.interleave_gate_up(q) if interleave else q,
                                 quant.interleave_gate_up(sf) if interleave else sf, vec)
    pair = mm.transform_weights_for_mega_moe((q, sf), (q, sf))[0 if interleave else 1]
    assert pair[1].tolist() == [512, 1024, vec]
    assert torch.equal(pair[0], want)
    # fp32 scales [E, N, K / vec] instead of packed words: same stream
    sf_bytes = sf.contiguous().view(torch.uint8).view(3, 512, -1)
    sf_f32 = sf_bytes.view(torch.float8_e4m3fn).float() if fmt == 'nvfp4' else (sf_bytes.to(torch.int32) << 23).view(torch.float32)
    pair32 = mm.transform_weights_for_mega_moe((q, sf_f32), (q, sf_f32))[0 if interleave else 1]
    assert torch.equal(pair32[0], want)


def test_transform_kernel_rate_on_the_full_layer():
    """48 experts x [2560, 3072]: a pure copy (reads and writes the weights once)."""
    q, sf = _weights('mxfp4', 48, 2560, 3072, 8)
    mm.transform_weights_for_mega_moe((q, sf), (q, sf))
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    out = mm.transform_weights_for_mega_moe((q, sf), (q, sf))
    t1.record()
    torch.cuda.synchronize()
    nbytes = 2 * 2 * (q.numel() + sf.numel() * 4)              # two layers' worth in this call, read + written
    gbs = nbytes / (t0.elapsed_time(t1) * 1e-3) / 1e9
    print(f'transform_weights: {nbytes / 1e6:.0f} MB moved in {t0.elapsed_time(t1):.3f} ms = {gbs:.0f} GB/s')
    assert out[0][0].shape == (48, 20, 12, 17408) and gbs > 1000


def test_fp4_cast_kernel_matches_the_reference_helper_vectors():
    lib = _lib.load()
    gold = np.load(os.path.join(GOLDEN, 'quant_helpers.npz'))
    x = torch.from_numpy(gold['x_bf16_as_f32']).to(torch.bfloat16).cuda()
    m, k = x.shape
    packed = torch.zeros((m, k // 2), dtype=torch.uint8, device='cuda')
    sf = torch.zeros((m, k // 32), dtype=torch.float32, device='cuda')
    st = lib.mm_cast_rows_to_fp4(x.data_ptr(), 1, m, k, 32, 1, packed.data_ptr(), sf.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert np.array_equal(packed.cpu().numpy(), gold['cast_fp4_packed'])
    assert np.array_equal(sf.cpu().numpy(), gold['cast_fp4_sf'])
    # fp32 input, same values
    xf = x.float()
    packed.zero_(); sf.zero_()
    assert lib.mm_cast_rows_to_fp4(xf.data_ptr(), 0, m, k, 32, 1, packed.data_ptr(), sf.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert np.array_equal(packed.cpu().numpy(), gold['cast_fp4_packed'])


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_global_scale_calibration_matches_torch(dtype):
    """`mm_tensor_absmax` / `nvfp4_global_scale`: largest magnitude of a tensor (sizes that are not multiples of the 16 B
    load, the maximum in the ragged tail, an all-zero and an empty tensor), exact against torch."""
    g = torch.Generator().manual_seed(5)
    for n in (1, 7, 4096, 48 * 2560 * 96 + 3):
        x = torch.randn(n, generator=g).to(dtype).cuda()
        if n > 4:
            x[-1] = 37.5                                  # in the tail beyond the last full 16 B load
        assert mm.nvfp4_global_scale(x) == float(x.float().abs().max().item()) / (6.0 * 448.0)
    assert mm.nvfp4_global_scale(torch.zeros(64, dtype=dtype, device='cuda')) == 0.0
    assert mm.nvfp4_global_scale(torch.zeros(0, dtype=dtype, device='cuda')) == 0.0
