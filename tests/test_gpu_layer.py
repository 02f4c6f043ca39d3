"""GPU parity of the fused layer (one rank): the CUDA kernel through the C ABI against the CPU oracle.

Tolerances (stated by the task for floating point): relative RMSE <= 0.3 % and cosine >= 0.9999 per rank for y;
per-expert counts and the canonical slot order are exact.
"""
import pytest
import torch

import hopper_megamoe_basedondeepgemm_b200 as mm
from oracle import megamoe_oracle as O
from tests import util_moe as U

pytestmark = pytest.mark.gpu
REL_RMSE_TOL, COS_TOL = 3e-3, 0.9999


def run_layer(fmt, e_local, hidden, inter, topk, tokens, routing, engine, seed=0, clamp=10.0, std=0.05, num_sms=0,
              global_scales=True, masked_ratio=0.0, t_max=None):
    dev = 'cuda'
    w, gs1, gs2 = O.make_expert_weights(e_local, hidden, inter, fmt, seed=seed + 17, std=std)
    if routing == 'balanced':
        idx, tw = O.balanced_routing(tokens, 0, 1, e_local, topk)
    else:
        idx, tw = U.random_routing(tokens, e_local, topk, seed + 3, masked_ratio)
    x_gs = 1.0
    mid_gs = 1.0
    if global_scales and fmt == 'nvfp4':
        x_gs, mid_gs = 1.0 / 64.0, 1.0 / 512.0
    x, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, seed + 5, idx, tw, x_global_scale=x_gs)
    ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=clamp, faithful=True, rounding='rne', keep_mid=True,
                                x_global_scale=x_gs, w1_global_scale=gs1, w2_global_scale=gs2, mid_global_scale=mid_gs)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, t_max or max(tokens, 1), topk, hidden, inter, act_format=fmt,
                                          num_sms=num_sms)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    U.write_inputs(buf, inp, sfb)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
    stats = torch.full((e_local,), 7, dtype=torch.int32, device=dev)
    if fmt == 'fp8':
        mm.fp8_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=clamp,
                            fast_math=True, engine=engine, timeout_ms=500.0)
    else:
        mm.fp4_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=clamp,
                            fast_math=True, engine=engine, x_global_scale=x_gs, l1_global_scale=gs1,
                            l2_global_scale=gs2, mid_global_scale=mid_gs, timeout_ms=500.0)
    st, words = buf.device_status()
    assert st == 0, f'device status {st}: {[hex(v) for v in words[:4]]} {U.last_cuda_error()}'
    return y.cpu(), stats.cpu(), ref, buf, inp


def check_against_oracle(y, stats, ref, buf, fmt, inter):
    assert torch.equal(stats - 7, ref.counts[0])                         # per-expert counts: exact
    if y.numel():
        assert O.rel_rmse(y, ref.y[0]) <= REL_RMSE_TOL, O.rel_rmse(y, ref.y[0])
        assert O.cosine(y, ref.y[0]) >= COS_TOL
    # slot map: the (expert, token, slot) records the kernel kept in the receive pool, grouped per expert in row order,
    # equal the canonical (source rank, token, slot) order exactly
    recs = buf.received_records()
    assert all(r is not None and all(v is not None for v in r) for r in recs)
    got_map = [[] for _ in ref.slot_map[0]]
    for src, rows in enumerate(recs):
        for (e, t, s, w) in rows:
            got_map[e].append((src, t, s))
    assert got_map == [list(v) for v in ref.slot_map[0]]
    # the intermediate rows of every expert sit in that order: row n of the pool is the oracle's row n (the values
    # themselves are floating-point results of a different summation order: almost all quantised codes agree)
    vec = O.SF_VEC[fmt]
    base, step = 0, buf.tile_image_rows() or 16              # rows of an expert start on a tile boundary (16 or 32 rows)
    mid = buf.l2_acts_payload().cpu()
    mid_sf = buf.l2_acts_sf_payload().cpu()
    mismatched = total = 0
    for e, cnt in enumerate(ref.counts[0].tolist()):
        if cnt == 0:
            continue
        got_q = mid[base:base + cnt]
        got_sf = mid_sf[base:base + cnt, :inter // vec]
        deq = O.dequant_fp8_rows if fmt == 'fp8' else (lambda q, sf: O.dequant_fp4_rows(q, sf, vec))
        want = deq(ref.mid_q[0][e], O.sf_bytes_to_float(ref.mid_sf[0][e], fmt))
        got = deq(got_q, O.sf_bytes_to_float(got_sf, fmt))
        for n in range(cnt):                                             # every row against its own reference row
            assert O.rel_rmse(got[n], want[n]) < 0.05, (e, n, O.rel_rmse(got[n], want[n]))
        mismatched += int((got != want).sum())
        total += want.numel()
        base += (cnt + step - 1) // step * step
    assert mismatched <= 0.01 * total, (mismatched, total)


@pytest.mark.parametrize('engine', ['check', 'umma'])
@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4'])
def test_small_layer(engine, fmt):
    y, stats, ref, buf, _ = run_layer(fmt, e_local=4, hidden=512, inter=256, topk=2, tokens=5, routing='random', engine=engine)
    check_against_oracle(y, stats, ref, buf, fmt, 256)


def test_small_layer_fp8_activations():
    y, stats, ref, buf, _ = run_layer('fp8', e_local=4, hidden=512, inter=256, topk=2, tokens=5, routing='random', engine='umma')
    check_against_oracle(y, stats, ref, buf, 'fp8', 256)


def test_many_rows_fp8_activations():
    y, stats, ref, buf, _ = run_layer('fp8', e_local=4, hidden=1024, inter=512, topk=3, tokens=40, routing='random',
                                      engine='umma', masked_ratio=0.2)
    check_against_oracle(y, stats, ref, buf, 'fp8', 512)


def test_full_shape_fp8_activations():
    y, stats, ref, buf, _ = run_layer('fp8', e_local=48, hidden=3072, inter=1280, topk=8, tokens=8, routing='balanced',
                                      engine='umma', std=0.02)
    check_against_oracle(y, stats, ref, buf, 'fp8', 1280)


@pytest.mark.parametrize('engine', ['check', 'umma'])
def test_many_rows_per_expert_and_masked_slots(engine):
    # 40 tokens x top-3 over 3 experts: up to 40 rows per expert -> three 16-row tiles; some slots masked (-1)
    y, stats, ref, buf, _ = run_layer('mxfp4', e_local=4, hidden=512, inter=256, topk=3, tokens=40, routing='random',
                                      engine=engine, masked_ratio=0.2)
    check_against_oracle(y, stats, ref, buf, 'mxfp4', 256)


@pytest.mark.parametrize('engine', ['check', 'umma'])
def test_zero_tokens(engine):
    y, stats, ref, buf, _ = run_layer('mxfp4', e_local=4, hidden=512, inter=256, topk=2, tokens=0, routing='random', engine=engine)
    assert torch.equal(stats - 7, torch.zeros(4, dtype=torch.int32))


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4'])
def test_full_shape_single_rank(fmt):
    """48 local experts, H=3072, I=1280, top-8, 8 tokens (the CPU-runnable configuration of the benchmark)."""
    y, stats, ref, buf, _ = run_layer(fmt, e_local=48, hidden=3072, inter=1280, topk=8, tokens=8, routing='balanced',
                                      engine='umma', std=0.02, global_scales=(fmt == 'nvfp4'))
    check_against_oracle(y, stats, ref, buf, fmt, 1280)


def test_engines_agree_on_full_shape():
    y1, _, _, _, _ = run_layer('mxfp4', 48, 3072, 1280, 8, 4, 'balanced', 'umma', std=0.02)
    y2, _, _, _, _ = run_layer('mxfp4', 48, 3072, 1280, 8, 4, 'balanced', 'check', std=0.02)
    assert O.rel_rmse(y1, y2) < 2e-3


def test_repeated_launches_alternate_parity():
    dev = 'cuda'
    fmt, e_local, hidden, inter, topk = 'mxfp4', 4, 512, 256, 2
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=1, std=0.05)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, topk, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    for it, tokens in enumerate([3, 16, 0, 7, 1]):
        idx, tw = U.random_routing(tokens, e_local, topk, 100 + it)
        x, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 200 + it, idx, tw)
        ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=None, faithful=True)
        U.write_inputs(buf, inp, sfb)
        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=None, timeout_ms=500.0)
        st, words = buf.device_status()
        assert st == 0 and words[1] == it + 1
        if tokens:
            assert O.rel_rmse(y.cpu(), ref.y[0]) <= REL_RMSE_TOL


def test_launch_inside_a_cuda_graph():
    """The launch is one kernel on the current stream with all per-launch state on the device (launch counters in the
    buffer): captured once, it replays on new inputs, as the reference's serving path does."""
    dev = 'cuda'
    fmt, e_local, hidden, inter, topk, tokens = 'mxfp4', 4, 512, 256, 2, 7
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=1, std=0.05)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, topk, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
    idx, tw = U.random_routing(tokens, e_local, topk, 500)
    _, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 501, idx, tw)
    U.write_inputs(buf, inp, sfb)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):                                   # warm-up launch outside the capture
        mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=None, timeout_ms=500.0)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=None, timeout_ms=500.0)
    for it in range(3):
        idx, tw = U.random_routing(tokens, e_local, topk, 510 + it)
        _, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 520 + it, idx, tw)
        ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=None, faithful=True)
        U.write_inputs(buf, inp, sfb)
        graph.replay()
        torch.cuda.synchronize()
        assert buf.device_status()[0] == 0
        assert O.rel_rmse(y.cpu(), ref.y[0]) <= REL_RMSE_TOL


def test_inputs_through_the_pinned_host_mirror():
    """All four input views arrive with one host-to-device copy of the buffer's input region."""
    dev = 'cuda'
    fmt, e_local, hidden, inter, topk, tokens = 'fp8', 4, 512, 256, 2, 6
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=1, std=0.05)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, topk, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    idx, tw = U.random_routing(tokens, e_local, topk, 77)
    x, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 78, idx, tw)
    ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=None, faithful=True)
    mirror, views = buf.host_inputs()
    views['x'][:tokens].copy_(inp.x_q.view(views['x'].dtype))
    views['x_sf'][:tokens].copy_(sfb.contiguous().view(torch.int32))
    views['topk_idx'][:tokens].copy_(inp.topk_idx)
    views['topk_weights'][:tokens].copy_(inp.topk_weights)
    buf.inputs.copy_(mirror, non_blocking=True)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
    mm.fp8_fp4_mega_moe(y, l1, l2, buf, activation_clamp=None, timeout_ms=500.0)
    assert buf.device_status()[0] == 0
    assert O.rel_rmse(y.cpu(), ref.y[0]) <= REL_RMSE_TOL


def test_reset_restarts_the_launch_numbering():
    """Words that cross between ranks are marked with the launch number. `reset` restarts the numbering, so it must
    also clear every marked word: after it, launch 1's stale rows (other tokens, other routing) must not be taken for
    current ones."""
    dev = 'cuda'
    fmt, e_local, hidden, inter, topk = 'mxfp4', 4, 512, 256, 2
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=1, std=0.05)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, topk, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    for it, tokens in enumerate([16, 9, 16, 5]):
        if it == 2:
            buf.reset()
        idx, tw = U.random_routing(tokens, e_local, topk, 300 + it)
        x, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 400 + it, idx, tw)
        ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=None, faithful=True)
        U.write_inputs(buf, inp, sfb)
        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=None, timeout_ms=500.0)
        st, words = buf.device_status()
        assert st == 0 and words[1] == (it % 2) + 1
        assert O.rel_rmse(y.cpu(), ref.y[0]) <= REL_RMSE_TOL


def test_bounded_wait_reports_timeout_and_buffer_recovers():
    """A dispatch flag that nothing sets: a two-rank configuration whose second rank never launches. The wait runs
    out after the budget, the status word says which wait, the context stays usable, and after a reset the buffer works."""
    import ctypes
    from hopper_megamoe_basedondeepgemm_b200 import _lib
    dev = 'cuda'
    fmt, e_local, hidden, inter, topk = 'mxfp4', 2, 512, 256, 2
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=1, std=0.05)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, topk, hidden, inter, act_format=fmt)
    lib = _lib.load()
    cfg2 = _lib.MMConfig(2, 0, 2 * e_local, 16, topk, hidden, inter, _lib.FMT[fmt], 0)
    L2 = _lib.MMLayout()
    assert lib.mm_get_layout(ctypes.byref(cfg2), ctypes.byref(L2)) == 0
    big = torch.zeros(int(L2.total_bytes), dtype=torch.int8, device=dev)
    peers = (ctypes.c_void_p * 2)(big.data_ptr(), big.data_ptr())
    y = torch.empty((0, hidden), dtype=torch.bfloat16, device=dev)
    args = _lib.MMLaunchArgs(big.data_ptr(), peers, l1[0].data_ptr(), l2[0].data_ptr(), None, 0, 0, None, -1.0, 1,
                             1.0, 1.0, 1.0, 1.0, 30.0, None)
    assert lib.mm_mega_moe_launch(ctypes.byref(cfg2), ctypes.byref(args), torch.cuda.current_stream().cuda_stream) == 0
    words = (ctypes.c_uint32 * 16)()
    st = lib.mm_read_device_status(ctypes.byref(cfg2), big.data_ptr(), words, torch.cuda.current_stream().cuda_stream)
    assert st == 4 and (words[0] & 0xFF) == 7 and (words[0] >> 16) == 1     # dispatch-flag wait, source rank 1
    # the context is alive and a healthy buffer still works
    idx, tw = U.random_routing(4, e_local, topk, 5)
    x, inp, sfb = U.make_rank_inputs(4, hidden, fmt, 6, idx, tw)
    ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=None)
    U.write_inputs(buf, inp, sfb)
    y = torch.empty((4, hidden), dtype=torch.bfloat16, device=dev)
    mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=None, timeout_ms=500.0)
    assert buf.device_status()[0] == 0
    assert O.rel_rmse(y.cpu(), ref.y[0]) <= REL_RMSE_TOL


@pytest.mark.parametrize('fmt', ['mxfp4', 'fp8'])
def test_kernel_features_do_not_change_the_result(fmt):
    """The scout's weight prefetch, the own-row listing, the early combine and the operand tile images (24 received rows
    here: more than one 16-row tile) are scheduling and data-movement changes only: with all of them off and with all of
    them on the layer writes the same bits."""
    from hopper_megamoe_basedondeepgemm_b200 import _lib
    lib = _lib.load()
    default = lib.mm_get_tuning(_lib.TUNE['knobs'])
    outs = []
    try:
        for knobs in (0, 7, 1, 2, 4, 16, 22, 54):            # (54 = 22 + the wait profile of the tile roles)
            mm.set_tuning(knobs=knobs)
            y, stats, ref, buf, _ = run_layer(fmt, e_local=48, hidden=3072, inter=1280, topk=8, tokens=3, routing='balanced',
                                              engine='umma', std=0.02)
            check_against_oracle(y, stats, ref, buf, fmt, 1280)
            outs.append(y)
    finally:
        mm.set_tuning(knobs=default)
    for y in outs[1:]:
        assert torch.equal(y, outs[0])


def test_inputs_read_from_pinned_host_memory_and_output_written_there():
    """`host_inputs`: the kernel reads x / x_sf / topk_idx / topk_weights straight from the pinned mirror and writes y
    to a pinned host tensor; the result equals the launch that works from the device views."""
    dev = 'cuda'
    fmt, e_local, hidden, inter, topk, tokens = 'mxfp4', 8, 1024, 512, 4, 5
    w, _, _ = O.make_expert_weights(e_local, hidden, inter, fmt, seed=1, std=0.05)
    buf = mm.get_symm_buffer_for_mega_moe(None, e_local, 16, topk, hidden, inter, act_format=fmt)
    l1, l2 = mm.transform_weights_for_mega_moe(*U.to_operator_weights(w, fmt, dev))
    idx, tw = U.random_routing(tokens, e_local, topk, 91, masked_ratio=0.1)
    _, inp, sfb = U.make_rank_inputs(tokens, hidden, fmt, 92, idx, tw)
    U.write_inputs(buf, inp, sfb)
    y_dev = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
    mm.fp4_fp4_mega_moe(y_dev, l1, l2, buf, activation_clamp=10.0, timeout_ms=500.0)
    assert buf.device_status()[0] == 0
    buf.inputs.zero_()                                                # the device views no longer hold the inputs
    mirror, views = buf.host_inputs()
    views['x'][:tokens].copy_(inp.x_q.view(views['x'].dtype))
    views['x_sf'][:tokens].copy_(sfb.contiguous().view(torch.int32))
    views['topk_idx'][:tokens].copy_(inp.topk_idx)
    views['topk_weights'][:tokens].copy_(inp.topk_weights)
    y_host = torch.zeros((tokens, hidden), dtype=torch.bfloat16).pin_memory()
    mm.fp4_fp4_mega_moe(y_host, l1, l2, buf, activation_clamp=10.0, timeout_ms=500.0, host_inputs=mirror)
    assert buf.device_status()[0] == 0                                # (synchronises: y_host is complete)
    assert torch.equal(y_host, y_dev.cpu())
    ref = O.moe_layer_reference([inp], [w], fmt, e_local, clamp=10.0)
    assert O.rel_rmse(y_host, ref.y[0]) <= REL_RMSE_TOL


def test_phase_stamps_are_ordered():
    y, stats, ref, buf, _ = run_layer('mxfp4', 48, 3072, 1280, 8, 1, 'balanced', 'umma', std=0.02)
    s = buf.phase_stamps()
    assert s[12] and s[12] <= s[0] + 50_000 and s[12] <= s[5] <= s[3] <= s[8]       # earliest entry, prologue, scheduled, last exit
    assert s[13] and s[12] <= s[13] <= s[14] <= s[8]                               # weight stream window inside the launch
    assert (s[8] - s[12]) < 5_000_000
