"""Router frontend on the GPU against the oracle: top-8 indices and quantised tokens bit-exact, weights to 1e-6."""
import pytest
import torch

import hopper_megamoe_basedondeepgemm_b200 as mm
from oracle import megamoe_oracle as O
from tests import util_moe as U

pytestmark = pytest.mark.gpu


def _canon(packed, fmt='mxfp4'):
    """-0 and +0 are the same value: clear the sign of zero nibbles (E2M1) or bytes (E4M3) before comparing."""
    u = packed.view(torch.uint8).clone()
    if fmt == 'fp8':
        u[u == 0x80] = 0
        return u
    lo, hi = u & 0xF, u >> 4
    lo[lo == 8] = 0
    hi[hi == 8] = 0
    return lo | (hi << 4)


def _run_frontend(fmt, tokens, num_experts, hidden, score_mode=0, bias=None, seed=0, x_gs=1.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    if tokens > 2:
        x[1] = 0                                                      # an all-zero token row
    wr = (torch.randn((num_experts, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    buf = mm.get_symm_buffer_for_mega_moe(None, num_experts, max(tokens, 16), 8, hidden, 1280, act_format=fmt)
    return x, wr, buf


def test_frontend_384_experts_through_the_c_abi():
    """The 8-rank routing width (384 experts) on one GPU: the frontend only needs this rank's buffer."""
    import ctypes
    from hopper_megamoe_basedondeepgemm_b200 import _lib
    lib = _lib.load()
    tokens, num_experts, hidden = 4, 384, 3072
    g = torch.Generator().manual_seed(21)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    wr = (torch.randn((num_experts, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    cfg = _lib.MMConfig(8, 0, num_experts, 16, 8, hidden, 1280, _lib.FMT['mxfp4'], 0)
    L = _lib.MMLayout()
    assert lib.mm_get_layout(ctypes.byref(cfg), ctypes.byref(L)) == 0
    buf = torch.zeros(int(L.total_bytes), dtype=torch.uint8, device='cuda')
    ws = torch.zeros(int(lib.mm_frontend_workspace_bytes(ctypes.byref(cfg))), dtype=torch.uint8, device='cuda')
    xd, wd = x.cuda(), wr.cuda()
    args = _lib.MMFrontendArgs(xd.data_ptr(), wd.data_ptr(), None, tokens, 0, ws.data_ptr(), 1.0)
    assert lib.mm_frontend_launch(ctypes.byref(cfg), buf.data_ptr(), ctypes.byref(args),
                                  torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    logits = O.router_logits_device_order(x, wr)
    idx, w = O.route_from_logits(logits, x, 8)
    got_idx = buf[L.off_topk_idx:L.off_topk_idx + tokens * 64].view(torch.int64).view(tokens, 8).cpu()
    got_w = buf[L.off_topk_weights:L.off_topk_weights + tokens * 32].view(torch.float32).view(tokens, 8).cpu()
    assert torch.equal(got_idx, idx)
    assert torch.allclose(got_w, w, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4', 'fp8'])
@pytest.mark.parametrize('score_mode', [0, 1])
def test_frontend_matches_oracle(fmt, score_mode):
    tokens, num_experts, hidden = 9, 48, 3072
    x, wr, buf = _run_frontend(fmt, tokens, num_experts, hidden, seed=3 + score_mode)
    bias = None
    if score_mode == 1:
        ranks = torch.arange(1, num_experts + 1, dtype=torch.float32)
        bias = (0.2 / ranks ** 1.2)[torch.randperm(num_experts, generator=torch.Generator().manual_seed(5))]
    ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
    x_gs = 1.0 / 64.0 if fmt == 'nvfp4' else 1.0
    mm.fe_forward_into_buffer(x.cuda(), wr.cuda(), buf, ws, score_mode=score_mode,
                              expert_bias=bias.cuda() if bias is not None else None, x_global_scale=x_gs)
    torch.cuda.synchronize()
    # the workspace holds 16 B per (token, expert): {first-half sum, flag, second-half sum, flag}
    parts = ws[256:256 + tokens * num_experts * 16].view(torch.float32).view(tokens, num_experts, 4).cpu()
    logits_gpu = (parts[..., 0] + parts[..., 2]).to(torch.bfloat16).float() + 0.0
    logits = O.router_logits_device_order(x, wr)
    assert torch.equal(logits_gpu, logits.float())                    # bit-exact logits
    idx, w = O.route_from_logits(logits, x, 8, 'softmax' if score_mode == 0 else 'sigmoid_bias', bias)
    assert torch.equal(buf.topk_idx[:tokens].cpu(), idx)              # bit-exact top-8, tie rule included
    assert torch.allclose(buf.topk_weights[:tokens].cpu(), w, rtol=2e-6, atol=1e-7)
    assert buf.topk_idx[1].tolist() == [-1] * 8 and float(buf.topk_weights[1].abs().sum()) == 0.0
    # value-level agreement with the reference's torch rule (fp32 matmul -> bf16): same experts for (almost) every token
    idx_ref, _, _ = O.router_reference(x, wr, 8, 'softmax' if score_mode == 0 else 'sigmoid_bias', bias)
    same = sum(set(a.tolist()) == set(b.tolist()) for a, b in zip(idx, idx_ref))
    assert same >= tokens - 1
    # quantised tokens
    q, sf, sfb = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul', global_scale=x_gs)
    assert torch.equal(_canon(buf.x[:tokens].cpu(), fmt), _canon(q, fmt))
    got_sf = buf.x_sf[:tokens].cpu().contiguous().view(torch.uint8).view(tokens, -1)
    assert torch.equal(got_sf, sfb)


def test_frontend_then_layer_matches_oracle():
    fmt, tokens, e_local, hidden, inter = 'mxfp4', 6, 48, 3072, 1280
    g = torch.Generator().manual_seed(11)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    wr = (torch.randn((e_local, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=12, std=0.02)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, 8, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, 'cuda'))
    ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
    # the reference's call, argument for argument (`sm100_b200/fe_sm100/test_e2e_b200.py:204-231`): mode 3 = MXFP4
    mm.fe_forward(x.cuda(), wr.cuda(), buf.x, buf.x_sf, buf.topk_idx, buf.topk_weights, ws, 3, 1)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
    mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=10.0, timeout_ms=500.0)
    assert buf.device_status()[0] == 0
    logits = O.router_logits_device_order(x, wr)
    idx, tw = O.route_from_logits(logits, x, 8)
    q, sf, _ = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul')
    ref = O.moe_layer_reference([O.RankInput(q, sf, idx, tw)], [w], fmt, e_local, clamp=10.0)
    assert O.rel_rmse(y.cpu(), ref.y[0]) <= 3e-3 and O.cosine(y.cpu(), ref.y[0]) >= 0.9999


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4', 'fp8'])
def test_layer_from_hidden_states_in_one_kernel(fmt):
    """Router, top-8, quantisation, dispatch, both GEMMs and the combine in a single launch."""
    tokens, e_local, hidden, inter = 7, 48, 3072, 1280
    g = torch.Generator().manual_seed(31)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    x[2] = 0
    wr = (torch.randn((e_local, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    w, gs1, gs2 = O.make_expert_weights(e_local, hidden, inter, fmt, seed=32, std=0.02)
    x_gs, mid_gs = (1.0 / 64.0, 1.0 / 512.0) if fmt == 'nvfp4' else (1.0, 1.0)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, 8, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, 'cuda'))
    ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
    for _ in range(2):                                           # second launch: other parity, arrival counter carries on
        mm.mega_moe_from_hidden(y, x.cuda(), wr.cuda(), l1, l2, buf, ws, activation_clamp=10.0, x_global_scale=x_gs,
                                l1_global_scale=gs1, l2_global_scale=gs2, mid_global_scale=mid_gs, timeout_ms=500.0)
        st, words = buf.device_status()
        assert st == 0, [hex(v) for v in words[:4]]
    logits = O.router_logits_device_order(x, wr)
    idx, tw = O.route_from_logits(logits, x, 8)
    assert torch.equal(buf.topk_idx[:tokens].cpu(), idx)
    q, sf, sfb = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul', global_scale=x_gs)
    routed = (idx >= 0).any(dim=1)
    assert torch.equal(_canon(buf.x[:tokens].cpu(), fmt)[routed], _canon(q, fmt)[routed])
    ref = O.moe_layer_reference([O.RankInput(q, sf, idx, tw)], [w], fmt, e_local, clamp=10.0, x_global_scale=x_gs,
                                w1_global_scale=gs1, w2_global_scale=gs2, mid_global_scale=mid_gs)
    assert O.rel_rmse(y.cpu(), ref.y[0]) <= 3e-3 and O.cosine(y.cpu(), ref.y[0]) >= 0.9999
    assert float(y[2].float().abs().sum()) == 0.0                # the all-zero token routes nowhere


@pytest.mark.parametrize('tokens', [16, 64])
def test_skewed_routing_full_layer(tokens):
    """Sigmoid scores + Zipf(1.2) expert bias, renormalised top-8: hot experts receive many rows (several 16-token tiles)."""
    fmt, e_local, hidden, inter = 'mxfp4', 48, 3072, 1280
    g = torch.Generator().manual_seed(41)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    wr = (torch.randn((e_local, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    ranks = torch.arange(1, e_local + 1, dtype=torch.float32)
    bias = (1.0 / ranks ** 1.2)[torch.randperm(e_local, generator=g)]
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=42, std=0.02)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, tokens, 8, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, 'cuda'))
    ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
    stats = torch.zeros(e_local, dtype=torch.int32, device='cuda')
    mm.mega_moe_from_hidden(y, x.cuda(), wr.cuda(), l1, l2, buf, ws, cumulative_local_expert_recv_stats=stats,
                            activation_clamp=10.0, score_mode=1, expert_bias=bias.cuda(), timeout_ms=1000.0)
    st, words = buf.device_status()
    assert st == 0, [hex(v) for v in words[:4]]
    logits = O.router_logits_device_order(x, wr)
    idx, tw = O.route_from_logits(logits, x, 8, 'sigmoid_bias', bias)
    assert torch.equal(buf.topk_idx[:tokens].cpu(), idx)
    q, sf, _ = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul')
    ref = O.moe_layer_reference([O.RankInput(q, sf, idx, tw)], [w], fmt, e_local, clamp=10.0)
    assert torch.equal(stats.cpu(), ref.counts[0])
    assert int(ref.counts[0].max()) > 16 or tokens < 64          # the hot expert spans more than one token tile
    assert O.rel_rmse(y.cpu(), ref.y[0]) <= 3e-3 and O.cosine(y.cpu(), ref.y[0]) >= 0.9999


def test_router_agrees_with_the_reference_rule_on_thousands_of_tokens():
    """384 experts, 4096 seeded tokens: the kernel's top-8 is bit-exact against the restatement of its own summation
    order, and the number of tokens whose expert SET differs from the reference's torch rule (fp32 matmul -> bf16 ->
    stable descending sort, `tests/test_four_api_correctness.py:371-374`) is counted: two orders of one fp32 sum can
    round to different bf16 logits only for near-ties at the eighth place."""
    import ctypes
    from hopper_megamoe_basedondeepgemm_b200 import _lib
    lib = _lib.load()
    tokens, num_experts, hidden, chunk = 4096, 384, 3072, 64
    g = torch.Generator().manual_seed(20260805)
    wr = (torch.randn((num_experts, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    cfg = _lib.MMConfig(8, 0, num_experts, chunk, 8, hidden, 1280, _lib.FMT['mxfp4'], 0)
    L = _lib.MMLayout()
    assert lib.mm_get_layout(ctypes.byref(cfg), ctypes.byref(L)) == 0
    buf = torch.zeros(int(L.total_bytes), dtype=torch.uint8, device='cuda')
    ws = torch.zeros(int(lib.mm_frontend_workspace_bytes(ctypes.byref(cfg))), dtype=torch.uint8, device='cuda')
    wd = wr.cuda()
    set_diff = order_diff = exact_diff = 0
    for c0 in range(0, tokens, chunk):
        x = torch.randn((chunk, hidden), generator=g).to(torch.bfloat16)
        xd = x.cuda()
        args = _lib.MMFrontendArgs(xd.data_ptr(), wd.data_ptr(), None, chunk, 0, ws.data_ptr(), 1.0)
        assert lib.mm_frontend_launch(ctypes.byref(cfg), buf.data_ptr(), ctypes.byref(args),
                                      torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        got = buf[L.off_topk_idx:L.off_topk_idx + chunk * 64].view(torch.int64).view(chunk, 8).cpu()
        idx, _ = O.route_from_logits(O.router_logits_device_order(x, wr), x, 8)
        exact_diff += int((got != idx).any(dim=1).sum())
        idx_ref, _, _ = O.router_reference(x, wr, 8)
        set_diff += sum(set(a.tolist()) != set(b.tolist()) for a, b in zip(got, idx_ref))
        order_diff += int((got != idx_ref).any(dim=1).sum())
    print(f'router: {tokens} tokens x {num_experts} experts: expert-set differences vs the reference rule {set_diff}, '
          f'order differences {order_diff}, differences vs the device-order restatement {exact_diff}')
    assert exact_diff == 0
    assert set_diff <= tokens // 100


def test_fused_frontend_after_other_launches_on_the_same_buffer():
    """A launch of the plain variant, or a fused launch without tokens, between fused launches must not disturb the
    frontend's arrival words: every launch waits for words carrying its own number."""
    fmt, e_local, hidden, inter, tokens = 'mxfp4', 8, 1024, 512, 5
    g = torch.Generator().manual_seed(51)
    x = torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)
    wr = (torch.randn((e_local, hidden), generator=g) / hidden ** 0.5).to(torch.bfloat16)
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=52, std=0.05)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, 8, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, 'cuda'))
    ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
    logits = O.router_logits_device_order(x, wr)
    idx, tw = O.route_from_logits(logits, x, 8)
    q, sf, sfb = O.quantise_tokens(x, fmt, rounding='rne', sf_rule='mul')
    inp = O.RankInput(q, sf, idx, tw)
    ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=10.0)
    xd, wd = x.cuda(), wr.cuda()

    def fused(n):
        y = torch.empty((n, hidden), dtype=torch.bfloat16, device='cuda')
        mm.mega_moe_from_hidden(y, xd[:n], wd, l1, l2, buf, ws, activation_clamp=10.0, timeout_ms=300.0)
        st, words = buf.device_status()
        assert st == 0, [hex(v) for v in words[:4]]
        return y

    def plain():
        U.write_inputs(buf, inp, sfb)
        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
        mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=10.0, timeout_ms=300.0)
        assert buf.device_status()[0] == 0
        return y
    for step in ('fused', 'plain', 'fused', 'fused0', 'fused', 'plain', 'plain', 'fused'):
        if step == 'fused0':
            fused(0)
            continue
        y = fused(tokens) if step == 'fused' else plain()
        assert O.rel_rmse(y.cpu(), ref.y[0]) <= 3e-3, step
