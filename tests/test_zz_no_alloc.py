"""The allocation-free entry point against the regular one.

`mm_mega_moe_launch_static_scratch` exists for hosts that are not allowed to allocate device memory when they call
the layer (a server that sized its GPU arena at start-up, a plugin inside another runtime's memory plan): it keeps
the layer's working memory in an array built into the library. Here it is called through the C ABI twice in a row
(the array keeps the first call's bytes, so the second call proves the clearing) and its output must match the
regular entry point, which works out of a caller-provided buffer, within the suite's parity tolerance. This file
sorts last on purpose: a failure here must not hide the other tests of a run that stops at the first failure.
"""
import ctypes

import pytest
import torch

import hopper_megamoe_basedondeepgemm_b200 as mm
from hopper_megamoe_basedondeepgemm_b200 import _lib
from oracle import megamoe_oracle as O
from tests import util_moe as U

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_regular_entry_twice():
    dev = 'cuda'
    lib = _lib.load()
    fmt, e_local, hidden, inter, topk, t_max = 'mxfp4', 8, 1024, 512, 4, 16
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=71, std=0.05)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, t_max, topk, hidden, inter, act_format=fmt)
    cfg = _lib.MMConfig(1, 0, e_local, t_max, topk, hidden, inter, _lib.FMT[fmt], 0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, tokens in enumerate([9, 4]):
        idx, tw = U.random_routing(tokens, e_local, topk, 300 + call, masked_ratio=0.1)
        _, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 400 + call, idx, tw)
        # regular entry point: inputs written into the caller's buffer views
        U.write_inputs(buf, inp, sfb)
        y_ref = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        mm.fp4_fp4_mega_moe(y_ref, l1, l2, buf, activation_clamp=10.0, timeout_ms=500.0)
        assert buf.device_status()[0] == 0
        # allocation-free entry point: plain device tensors in, y out; everything below was allocated beforehand
        x_d = inp.x_q.view(torch.int8).to(dev)
        sf_d = sfb.contiguous().to(dev)
        idx_d, tw_d = inp.topk_idx.to(dev), inp.topk_weights.to(dev)
        y = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=dev)
        status = torch.full((16,), 0xFFFF, dtype=torch.int32, device=dev)
        args = _lib.MMStaticArgs(x_d.data_ptr(), sf_d.data_ptr(), idx_d.data_ptr(), tw_d.data_ptr(),
                                 l1[0].data_ptr(), l2[0].data_ptr(), y.data_ptr(), tokens, 1, None, 10.0,
                                 1.0, 1.0, 1.0, 1.0, 500.0, status.data_ptr())
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        st = lib.mm_mega_moe_launch_static_scratch(ctypes.byref(cfg), ctypes.byref(args), stream)
        assert st == 0, lib.mm_last_cuda_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call > 0:                    # (the first call may load the kernel's module; from then on nothing is allocated)
            assert free_after == free_before, (free_before, free_after)
        assert int(status[0]) == 0, hex(int(status[0]))
        assert O.rel_rmse(y.cpu(), y_ref.cpu()) <= 3e-3 and O.cosine(y.cpu(), y_ref.cpu()) >= 0.9999
        ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=10.0)
        assert O.rel_rmse(y.cpu(), ref.y[0]) <= 3e-3


def test_static_scratch_entry_rejects_what_it_cannot_hold():
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    args = _lib.MMStaticArgs(None, None, None, None, None, None, None, 0, 1, None, -1.0, 1.0, 1.0, 1.0, 1.0, 0.0, None)
    big = _lib.MMConfig(1, 0, 48, 2048, 8, 3072, 1280, _lib.FMT['mxfp4'], 0)          # working memory beyond the array
    assert lib.mm_mega_moe_launch_static_scratch(ctypes.byref(big), ctypes.byref(args), stream) == 2
    assert b'static scratch holds' in lib.mm_last_cuda_error()
    two = _lib.MMConfig(2, 0, 16, 16, 4, 1024, 512, _lib.FMT['mxfp4'], 0)             # peers cannot reach the array
    assert lib.mm_mega_moe_launch_static_scratch(ctypes.byref(two), ctypes.byref(args), stream) == 2
