"""Benchmark of the fused MegaMoE layer: kernel microseconds per layer (max over ranks) and HBM roofline fraction.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--tokens-per-rank T] [--active-ranks 0,4]
                    [--format mxfp4|nvfp4|fp8] [--from-hidden] [--no-sweep] [--no-parity]

N = 1 runs the single-GPU configuration (48 local experts, the per-rank work of the 8-rank global-M=8 case: 8 routed
rows on 8 experts). Under torchrun (N > 1) every rank owns 48 experts and feeds T tokens (default 1), i.e. the
8-rank run is the reference's headline case E=384 / H=3072 / I=1280 / top-8 / global M=8; `--active-ranks` leaves the
other ranks without tokens (the reference harness's option of the same name, `sm100_b200/test_mega_moe.py:47-50`:
global M=2 is ranks 0,4 and M=4 ranks 0,1,4,5). One JSON line on rank 0. Outside the timed region the run checks the
kernel's output of the benchmarked configuration against the CPU oracle (all ranks' inputs gathered, every rank
evaluates its own experts, partial results all-reduced: the reference's `--torch-ref` method,
`sm100_b200/test_mega_moe.py:438-499`) and reports it as `parity`; a failed check makes the run exit non-zero.
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, TOPK, E_LOCAL = 3072, 1280, 8, 48
T_MAX = 16
DTYPE_NAME = {'mxfp4': 'fp4 (e2m1) x fp4, fp32 accumulate', 'nvfp4': 'fp4 (e2m1) x fp4, fp32 accumulate',
              'fp8': 'fp8 (e4m3) x fp4 (e2m1), fp32 accumulate'}
NVLINK_GBS = 900.0           # per direction per GPU (nominal), the figure the roofline definition names
NVLINK_RTT_US = 2.3          # one NVLink round trip as the reference measured it (docs/B200_MEGAMOE_RESULTS.md:115: 3 trips ~ 7 us)
REL_RMSE_TOL, COS_TOL = 3e-3, 0.9999


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured (MEASURED_PEAKS.json)'
    return 6650.0, 'fallback'


def recorded_traffic(fmt, n):
    """DRAM bytes per algorithmic byte from the committed ncu summary of this workload, if one exists: (ratio, source)."""
    path = os.path.join(ROOT, 'profiles', 'dram_traffic.txt')
    if n != 1 or not os.path.exists(path):
        return None, None
    with open(path) as f:
        for line in f:
            parts = line.split()
            if len(parts) >= 3 and not line.startswith('#') and parts[0] == fmt:
                return float(parts[1]), f'constant from profiles/dram_traffic.txt ({" ".join(parts[2:])}), not measured in this run'
    return None, None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML from a thread while the timed region runs (read-only queries)."""

    def __init__(self, gpu_index):
        self.gpu_index, self.samples, self.reasons, self.max_mhz = gpu_index, [], set(), None
        self._stop, self._thread = False, None

    def _loop(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            names = {'hw_slowdown': pynvml.nvmlClocksThrottleReasonHwSlowdown,
                     'hw_thermal_slowdown': pynvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                     'sw_thermal_slowdown': pynvml.nvmlClocksThrottleReasonSwThermalSlowdown,
                     'sw_power_cap': pynvml.nvmlClocksThrottleReasonSwPowerCap}
            while not self._stop:
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                r = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
                time.sleep(0.002)
        except Exception as ex:                       # NVML missing: report it, never fail the benchmark
            self.reasons.add(f'nvml unavailable: {type(ex).__name__}')

    def start(self):
        import threading
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=5)
        return {'sm_mhz': statistics.median(self.samples) if self.samples else None, 'sm_max_mhz': self.max_mhz,
                'reasons': sorted(self.reasons), 'samples': len(self.samples)}


def cpu_reference_us(tokens, fmt, reps, threads=None):
    """The reference's pure-torch quantised MoE (the CPU oracle port) on the host cores, microseconds per layer, in two
    variants: weights dequantised inside the timed call, and dequantised once beforehand (as the reference's test does,
    `sm100_b200/test_mega_moe.py:411-420`). Returns (us with dequantisation, us without, threads used)."""
    import torch
    from oracle import megamoe_oracle as O
    from tests import util_moe as U
    torch.set_num_threads(threads or os.cpu_count() or 1)
    w, gs1, gs2 = O.make_expert_weights(E_LOCAL, HIDDEN, INTER, fmt, seed=0, std=0.02)
    idx, tw = O.balanced_routing(max(tokens, 1), 0, 1, E_LOCAL, TOPK)
    _, inp, _ = U.make_rank_inputs(max(tokens, 1), HIDDEN, fmt, 1, idx, tw)
    vec_w = 32 if fmt == 'fp8' else O.SF_VEC[fmt]
    active = sorted({int(e) for e in idx.flatten().tolist() if e >= 0})
    deq = {(0, e): (O.dequant_fp4_rows(w.w1_q[e], w.w1_sf[e], vec_w) * gs1, O.dequant_fp4_rows(w.w2_q[e], w.w2_sf[e], vec_w) * gs2)
           for e in active}
    out = []
    for cache in (None, deq):
        times = []
        for i in range(reps + 1):
            t0 = time.perf_counter()
            O.moe_layer_reference([inp], [w], fmt, E_LOCAL, clamp=10.0, w1_global_scale=gs1, w2_global_scale=gs2,
                                  dequantised=cache)
            if i:
                times.append((time.perf_counter() - t0) * 1e6)
        out.append(statistics.median(times))
    return out[0], out[1], torch.get_num_threads()


def run_reference(args):
    if int(os.environ.get('RANK', '0')) != 0:
        return
    reps = max(args.steps, 3)
    us, us_pre, cores = cpu_reference_us(args.tokens_per_rank, args.format, reps)
    sample = (f'{reps} repetitions (after 1 warm-up) of one rank\'s layer: {max(args.tokens_per_rank, 1)} token(s) x top-8 '
              f'over 48 experts, H=3072, I=1280, {args.format}; weights dequantised inside the timed call '
              f'(with the weights dequantised beforehand: {us_pre:.0f} us)')
    line = {'impl': 'reference', 'metric': 'moe_layer_kernel_us', 'value': us, 'unit': 'us', 'n_gpus': args.gpus,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': us / 1e3, 'higher_is_better': False,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': DTYPE_NAME[args.format], 'data': 'synthetic',
            'config': workload_config(args, args.gpus, [args.tokens_per_rank] * args.gpus),
            'cpu_baseline': {'value': us, 'unit': 'us', 'cores': cores, 'kind': 'port', 'sample': sample,
                             'value_weights_predequantised': us_pre},
            'e2e': {'value': us, 'unit': 'us', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}
    print(json.dumps(line))


def workload_config(args, n, tokens):
    fmt_name = 'W4A8 (MXFP4 x FP8)' if args.format == 'fp8' else 'W4A4 ' + args.format.upper()
    routing = 'router-picked' if getattr(args, 'from_hidden', False) else 'forced-balanced'
    per_rank = f'{tokens[0]} token(s) per rank' if len(set(tokens)) == 1 else f'tokens per rank {tokens}'
    return {'workload': f'EP{n} {fmt_name} MegaMoE layer, E={E_LOCAL * n} ({E_LOCAL}/rank), H={HIDDEN}, I={INTER}, top-{TOPK}, '
                        f'{routing} routing, {per_rank} (global M={sum(tokens)}), weights ~N(0,0.02)'
                        + (', from bf16 hidden states: router GEMM, top-8 and token quantisation fused into the same kernel'
                           if getattr(args, 'from_hidden', False) else ''),
            'l2': 'flushed by a 256 MiB write before every timed step; then the inputs are copied into the buffer views',
            'parallelism': f'ep{n}'}


def sweep_cases(n):
    """Global-M cases of the metric, as tokens per rank: the reference's owner layout on 8 ranks
    (`docs/B200_MEGAMOE_RESULTS.md:18-20`), all ranks with 1 or 2 tokens otherwise."""
    if n == 8:
        return {'M2': [1 if r in (0, 4) else 0 for r in range(8)], 'M4': [1 if r in (0, 1, 4, 5) else 0 for r in range(8)],
                'M8': [1] * 8, 'M16': [2] * 8}
    return {f'M{n}': [1] * n, f'M{2 * n}': [2] * n}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--tokens-per-rank', type=int, default=1)
    ap.add_argument('--active-ranks', default='', help='comma-separated ranks that own tokens (default: all)')
    ap.add_argument('--format', default='mxfp4', choices=['mxfp4', 'nvfp4', 'fp8'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-sweep', action='store_true', help='skip the extra global-M cases (m_sweep)')
    ap.add_argument('--no-parity', action='store_true', help='skip the oracle check of the benchmarked configuration')
    ap.add_argument('--num-sms', type=int, default=0)
    ap.add_argument('--knobs', type=int, default=-1, help='kernel feature bit mask (mm_set_tuning), default: library default')
    ap.add_argument('--stages', type=int, default=0)
    ap.add_argument('--prefetch-experts', type=int, default=-1)
    ap.add_argument('--skewed', action='store_true',
                    help='with --from-hidden: sigmoid scores + Zipf(1.2) expert bias instead of softmax scores (hot experts)')
    ap.add_argument('--from-hidden', action='store_true',
                    help='time the single-kernel layer from bf16 hidden states (router + top-8 + quantisation fused in)')
    args = ap.parse_args()
    if args.impl == 'reference':
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import hopper_megamoe_basedondeepgemm_b200 as mm
    from hopper_megamoe_basedondeepgemm_b200 import workload as W

    rank, world = int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
        group = dist.group.WORLD
    n, fmt = world, args.format
    num_experts = E_LOCAL * n
    W_WARM = max(args.warmup, 3)
    if args.knobs >= 0:
        mm.set_tuning(knobs=args.knobs)
    if args.stages > 0:
        mm.set_tuning(stages=args.stages)
    if args.prefetch_experts >= 0:
        mm.set_tuning(prefetch_w1_experts=args.prefetch_experts, prefetch_w2_experts=args.prefetch_experts)

    buf = mm.get_symm_buffer_for_mega_moe(group, num_experts, max(T_MAX, args.tokens_per_rank), TOPK, HIDDEN, INTER, act_format=fmt,
                                          num_sms=args.num_sms)
    l1, l2, (gs1, gs2), raw_w = W.make_layer_weights(E_LOCAL, HIDDEN, INTER, fmt, seed=1000 + rank, keep_untransformed=True)
    x_gs, mid_gs = (1.0 / 64.0, 1.0 / 512.0) if fmt == 'nvfp4' else (1.0, 1.0)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device='cuda')
    align = torch.ones(1, device='cuda')
    h_in, h_views = buf.host_inputs()
    active_ranks = [int(v) for v in args.active_ranks.split(',') if v != ''] or list(range(n))
    main_tokens = [args.tokens_per_rank if r in active_ranks else 0 for r in range(n)]

    class Case:
        """One workload: tokens per rank -> this rank's inputs, routing, output tensors and launch closures."""

        def __init__(self, tokens):
            self.tokens, self.T = tokens, tokens[rank]
            T = self.T
            _, self.xq, self.xsf = W.make_tokens(T, HIDDEN, fmt, seed=2000 + rank, global_scale=x_gs)
            self.idx, self.tw = W.balanced_routing(T, rank, n, num_experts, TOPK, device='cuda')
            self.all_idx = [W.balanced_routing(tokens[r], r, n, num_experts, TOPK)[0] for r in range(n)]
            self.active = W.active_experts_per_rank(self.all_idx, num_experts, n)
            self.rows_out = T * TOPK
            self.y = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device='cuda')
            self.h_y = torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory()
            self.stats = torch.zeros(E_LOCAL, dtype=torch.int32, device='cuda')

        def write_inputs(self):
            T = self.T
            if T:
                buf.x[:T].copy_(self.xq); buf.x_sf[:T].copy_(self.xsf)
                buf.topk_idx[:T].copy_(self.idx); buf.topk_weights[:T].copy_(self.tw)

        def fill_host_mirror(self):
            T = self.T
            if T:
                h_views['x'][:T].copy_(self.xq.cpu()); h_views['x_sf'][:T].copy_(self.xsf.cpu())
                h_views['topk_idx'][:T].copy_(self.idx.cpu()); h_views['topk_weights'][:T].copy_(self.tw.cpu())

        def launch(self, y=None, host_inputs=None, stats=None):
            y = self.y if y is None else y
            if fmt == 'fp8':
                mm.fp8_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0,
                                    fast_math=True, host_inputs=host_inputs)
            else:
                mm.fp4_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0,
                                    fast_math=True, x_global_scale=x_gs, l1_global_scale=gs1, l2_global_scale=gs2,
                                    mid_global_scale=mid_gs, host_inputs=host_inputs)

    class HiddenCase(Case):
        """The single-kernel path from bf16 hidden states: the routing is whatever the router picks."""

        def __init__(self, tokens):
            super().__init__(tokens)
            g = torch.Generator(device='cuda').manual_seed(77)
            self.wr = (torch.randn((num_experts, HIDDEN), generator=g, device='cuda') / HIDDEN ** 0.5).to(torch.bfloat16)
            g = torch.Generator(device='cuda').manual_seed(3000 + rank)
            self.hidden_src = torch.randn((self.T, HIDDEN), generator=g, device='cuda').to(torch.bfloat16)
            self.hidden_dev = self.hidden_src.clone()
            self.h_hidden = self.hidden_src.cpu().pin_memory()
            self.ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
            # --skewed: sigmoid scores + Zipf(1.2) expert bias (a random permutation of 1 / rank^1.2 over all experts),
            # renormalised top-8: hot experts receive many rows, most experts few or none
            self.bias = None
            if args.skewed:
                gb = torch.Generator().manual_seed(11)
                self.bias = (1.0 / torch.arange(1, num_experts + 1, dtype=torch.float32) ** 1.2)[torch.randperm(num_experts, generator=gb)].cuda()
            if world > 1:
                dist.barrier()
            self.launch(stats=self.stats)
            torch.cuda.synchronize()
            mine = torch.tensor([int((self.stats > 0).sum())], device='cuda')
            if world > 1:
                gathered = [torch.zeros_like(mine) for _ in range(world)]
                dist.all_gather(gathered, mine)
                self.active = [int(v) for v in gathered]
            else:
                self.active = [int(mine)]
            self.stats.zero_()

        def write_inputs(self):
            self.hidden_dev.copy_(self.hidden_src)

        def launch(self, y=None, host_inputs=None, stats=None):
            mm.mega_moe_from_hidden(self.y if y is None else y, self.hidden_dev, self.wr, l1, l2, buf, self.ws,
                                    cumulative_local_expert_recv_stats=stats, activation_clamp=10.0, fast_math=True,
                                    score_mode=1 if self.bias is not None else 0, expert_bias=self.bias, x_global_scale=x_gs, l1_global_scale=gs1, l2_global_scale=gs2, mid_global_scale=mid_gs)

    def timed(step_fn, prep_fn, steps, warm, tag):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for _ in range(20):                        # let the host run ahead of the GPU: events then bracket the kernel,
            flush.zero_()                          # not the host's launch latency
        for i in range(warm + steps):
            if i == warm:
                torch.cuda.nvtx.range_push(tag)
            flush.zero_()
            if prep_fn is not None:
                prep_fn()                          # flush -> input copy -> rank alignment -> kernel, as the reference's
            if world > 1:                          # streamed replay does (sm100_b200/test_mega_moe.py:351-357)
                dist.all_reduce(align)
            if i >= warm:
                starts[i - warm].record()
            step_fn()
            if i >= warm:
                ends[i - warm].record()
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
        return [s.elapsed_time(e) * 1e3 for s, e in zip(starts, ends)]

    STAMP_NAMES = {1: 'dispatched', 2: 'dispatch_headers_seen', 3: 'scheduled', 4: 'tasks_done', 5: 'prologue_done', 7: 'exit',
                   8: 'last_sm_exit', 9: 'frontend_done', 10: 'last_sm_tasks_done', 11: 'last_sm_scheduled',
                   13: 'first_weight_request', 14: 'last_weight_landed', 0: 'sm0_first_instruction'}

    def device_spans(case, reps=10):
        """Device-side times (globaltimer) of a few extra launches: span = first instruction of the earliest SM to the
        last SM's exit; weight-stream window = first weight request to the last unit found in shared memory."""
        spans, windows, stamps = [], [], None
        for _ in range(reps):
            flush.zero_()
            case.write_inputs()
            if world > 1:
                dist.all_reduce(align)
            case.launch()
            stamps = buf.phase_stamps()
            spans.append((stamps[8] - stamps[12]) / 1e3)
            if stamps[13] and stamps[14] > stamps[13]:
                windows.append((stamps[14] - stamps[13]) / 1e3)
        phases = {name: round((stamps[i] - stamps[12]) / 1e3, 2) for i, name in sorted(STAMP_NAMES.items()) if stamps[i]}
        return statistics.median(spans), (statistics.median(windows) if windows else None), phases

    SM_PHASE_NAMES = ['entry', 'prologue', 'own_listed', 'counts_known', 'scheduled', 'first_issue', 'first_landed', 'first_staged',
                      'first_mma_done', 'first_epilogue', 'last_l1_epilogue', 'first_l2_staged', 'tasks_done', 'first_combined',
                      'combine_done', 'exit', 'rows_cached']

    def sm_phase_summary():
        """Per-SM phase times of the latest launch on this rank, relative to its earliest SM entry: {phase: [min, median, max]} us."""
        raw = buf.sm_phases()
        ph = torch.cat([raw[:, :16], raw[:, 31:32]], dim=1).double()
        live = ph[:, 0] > 0
        if not bool(live.any()):
            return None
        ph = ph[live]
        t0 = ph[:, 0].min()
        out = {}
        for i, name in enumerate(SM_PHASE_NAMES):
            col = ph[:, i]
            col = col[col >= t0]                           # (a slot no launch has written yet, or a stale earlier one: left out)
            if col.numel():
                v = ((col - t0) / 1e3)
                out[name] = [round(float(v.min()), 2), round(float(v.median()), 2), round(float(v.max()), 2)]
        if mm._lib.load().mm_get_tuning(mm._lib.TUNE['knobs']) & 32:
            # wait profile (knob 32): cycles the roles spent waiting, as us (cycle length from the MMA role's own two clocks)
            w = raw[live][:, 16:30].double()
            ns_per_cycle = (w[:, 9] / w[:, 4].clamp(min=1)).median()
            names = ['loader_waits_free_stage', 'mma_waits_tokens', 'mma_waits_accumulator', 'mma_waits_weights', 'mma_role',
                     'epilogue_waits_mma', 'epilogue_role', 'epilogue_l1_work', 'epilogue_l2_work', 'mma_role_ns', 'mma_waits_token_records', 'release_latency_sum', 'release_latency_max', 'release_busy']
            out['wait_profile_us_median_max'] = {n: [round(float((w[:, i] * ns_per_cycle / 1e3).median()), 2),
                                                     round(float((w[:, i] * ns_per_cycle / 1e3).max()), 2)] for i, n in enumerate(names)}
        return out

    def reduce_max(values):
        t = torch.tensor([(-1.0 if v is None else float(v)) for v in values], device='cuda', dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [None if v < 0 else v for v in t.tolist()]

    def check_status(where):
        st, words = buf.device_status()
        if st != 0:
            raise RuntimeError(f'{where}: device status {st}: {[hex(v) for v in words[:4]]}')

    def parity(case):
        """Oracle check of `case` on every rank (CPU torch maths of the reference's quantised MoE); dict for the JSON line."""
        from oracle import megamoe_oracle as O
        T_all = case.tokens
        tcap = max(max(T_all), 1)
        case.write_inputs()
        case.stats.zero_()
        if world > 1:
            dist.barrier()
        case.launch(stats=case.stats)
        check_status('parity launch')
        y_dev = case.y.clone()

        def gather(t, shape, dtype):
            mine = torch.zeros((tcap,) + shape, dtype=dtype, device='cuda')
            if case.T:
                mine[:case.T].copy_(t.view(dtype).view((case.T,) + shape))
            if world == 1:
                return [mine.cpu()]
            out = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(out, mine)
            return [o.cpu() for o in out]
        L = buf.layout
        xq = gather(buf.x[:case.T].contiguous(), (int(L.x_row_bytes),), torch.uint8)
        xsf = gather(buf.x_sf[:case.T].contiguous().view(torch.uint8), (int(L.x_sf_row_bytes),), torch.uint8)
        idx = gather(buf.topk_idx[:case.T].contiguous(), (TOPK,), torch.int64)
        tw = gather(buf.topk_weights[:case.T].contiguous(), (TOPK,), torch.float32)
        inputs = [O.RankInput(xq[r][:T_all[r]], O.sf_bytes_to_float(xsf[r][:T_all[r]], fmt), idx[r][:T_all[r]], tw[r][:T_all[r]])
                  for r in range(world)]
        smap = O.canonical_slot_map([i.topk_idx for i in inputs], num_experts)[rank]
        wfmt = 'mxfp4' if fmt == 'fp8' else fmt
        (w1, w1_sf), (w2, w2_sf) = raw_w
        local = {}
        for e in range(E_LOCAL):
            if smap[e]:
                local[e] = (w1[e].cpu().view(torch.uint8), O.sf_bytes_to_float(w1_sf[e].contiguous().view(torch.uint8).cpu(), wfmt),
                            w2[e].cpu().view(torch.uint8), O.sf_bytes_to_float(w2_sf[e].contiguous().view(torch.uint8).cpu(), wfmt))
        routes, counts, _ = O.moe_rank_routes(inputs, local, rank, fmt, num_experts, clamp=10.0, x_global_scale=x_gs,
                                              w1_global_scale=gs1, w2_global_scale=gs2, mid_global_scale=mid_gs)
        part = torch.zeros((world, tcap, TOPK, HIDDEN), dtype=torch.float32)
        for (src, t, s), row in routes.items():
            part[src, t, s] = row
        part = part.cuda()
        if world > 1:
            dist.all_reduce(part)                  # exactly one rank contributes a non-zero row per (source, token, slot)
        y_ref = torch.zeros((case.T, HIDDEN), dtype=torch.float32)
        mine = part[rank].cpu()
        for t in range(case.T):
            for s in range(TOPK):                  # ascending slot order, fp32, one bf16 rounding at the end
                if int(inputs[rank].topk_idx[t, s]) >= 0:
                    y_ref[t] += mine[t, s]
        y_ref = y_ref.to(torch.bfloat16)
        rel = O.rel_rmse(y_dev.cpu(), y_ref) if case.T else 0.0
        cos = O.cosine(y_dev.cpu(), y_ref) if case.T else 1.0
        counts_ok = bool(torch.equal(case.stats.cpu(), counts))
        # slot map: the (expert, token, slot) records the kernel kept in the receive pool, grouped per expert in row
        # order, against the canonical (source rank, token, slot) order: exact
        recs = buf.received_records()
        got = [[] for _ in range(E_LOCAL)]
        slots_ok = all(r is not None and all(v is not None for v in r) for r in recs)
        if slots_ok:
            for src, rows in enumerate(recs):
                for (e, t, s, _) in rows:
                    got[e].append((src, t, s))
            slots_ok = got == [list(v) for v in smap]
        # from bf16 hidden states: the routing the kernel's frontend wrote against the oracle's router on the same tokens
        # (bf16 logits in the kernel's summation order, top-8 by value then expert index): exact
        top8_ok = True
        if isinstance(case, HiddenCase) and case.T:
            hx, wr = case.hidden_src.cpu(), case.wr.cpu()
            mode = 'sigmoid_bias' if case.bias is not None else 'softmax'
            idx_ref, _ = O.route_from_logits(O.router_logits_device_order(hx, wr), hx, TOPK, mode,
                                             None if case.bias is None else case.bias.cpu())
            top8_ok = bool(torch.equal(inputs[rank].topk_idx, idx_ref))
        flags = torch.tensor([rel, -cos, 0.0 if counts_ok else 1.0, 0.0 if slots_ok else 1.0, 0.0 if top8_ok else 1.0],
                             device='cuda', dtype=torch.float64)
        if world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.MAX)
        rel, ncos, cbad, sbad, tbad = flags.tolist()
        extra = {'top8_exact': tbad == 0.0, 'rows_per_expert_max_this_rank': int(counts.max())} if isinstance(case, HiddenCase) else {}
        if tbad != 0.0:
            cbad = 1.0
        return {**extra, 'rel_rmse_max_over_ranks': rel, 'cosine_min_over_ranks': -ncos, 'counts_exact': cbad == 0.0,
                'slot_map_exact': sbad == 0.0, 'tolerance': {'rel_rmse': REL_RMSE_TOL, 'cosine': COS_TOL},
                'shape': f'E={num_experts}, H={HIDDEN}, I={INTER}, top-{TOPK}, tokens per rank {T_all}, {fmt}',
                'checker': 'CPU oracle (pure-torch quantised MoE), every rank its own experts, partial outputs all-reduced',
                'ok': rel <= REL_RMSE_TOL and -ncos >= COS_TOL and cbad == 0.0 and sbad == 0.0}

    def nvlink_bytes(case):
        """Bytes this rank sends over NVLink per launch: its rows routed to other ranks (flagged words double the
        payload) and the header lines, plus the bf16 expert outputs it returns for the rows other ranks sent it."""
        L = buf.layout
        if world == 1:
            return 0
        dest = [torch.div(i[i >= 0], E_LOCAL, rounding_mode='floor') for i in case.all_idx]
        rows_out = int((dest[rank] != rank).sum())
        rows_back = sum(int((dest[r] == rank).sum()) for r in range(world) if r != rank)
        return int(rows_out * 2 * int(L.rx_row_bytes) + (world - 1) * 32 + rows_back * HIDDEN * 4)

    def steady_state(case, steps=48):
        """The same workload without the L2 flush, with the routed experts rotating from step to step (six disjoint groups
        of eight per rank: 300 MB of weights, so a group's weights have left the 126 MB L2 before it comes round again,
        while the kernel's code stays cached): what consecutive layers of a serving loop see. (event us, span us)."""
        variants = [W.balanced_routing(case.T, rank, n, num_experts, TOPK, token_offset=8 * k if n > 1 else k, device='cuda')[0]
                    for k in range(6)]
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        spans = []
        for _ in range(20):
            flush.zero_()
        for i in range(6 + steps):
            case.write_inputs()
            if case.T:
                buf.topk_idx[:case.T].copy_(variants[i % 6])
            if world > 1:
                dist.all_reduce(align)
            if i >= 6:
                starts[i - 6].record()
            case.launch()
            if i >= 6:
                ends[i - 6].record()
        torch.cuda.synchronize()
        ev = [a.elapsed_time(b) * 1e3 for a, b in zip(starts, ends)]
        for i in range(8):
            case.write_inputs()
            if case.T:
                buf.topk_idx[:case.T].copy_(variants[i % 6])
            if world > 1:
                dist.all_reduce(align)
            case.launch()
            st_ = buf.phase_stamps()
            spans.append((st_[8] - st_[12]) / 1e3)
        case.write_inputs()
        return sum(ev) / len(ev), statistics.median(spans)

    main_case = HiddenCase(main_tokens) if args.from_hidden else Case(main_tokens)
    main_case.write_inputs()
    sampler = ClockSampler(local)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    t_wall0 = time.perf_counter()
    ks = timed(main_case.launch, main_case.write_inputs, args.steps, W_WARM, 'timed')
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall0
    clocks = sampler.stop() if rank == 0 else None
    check_status('timed region')
    span_us, window_us, phases = device_spans(main_case)
    check_status('span launches')
    sm_summary = sm_phase_summary()

    # event-timing floor: two events with nothing / with a one-element kernel between them (what any launch pays)
    floor = timed(lambda: None, None, 20, 3, 'floor_empty')
    floor_k = timed(lambda: align.add_(0.0), None, 20, 3, 'floor_kernel')

    # end-to-end leg, two ways. (a) copies: the step's inputs sit in one pinned host mirror of the buffer's input region
    # and reach the device with a single copy; y comes back to pinned memory with another. (b) mapped: the kernel reads
    # the inputs straight from the pinned mirror and writes y straight to pinned memory: one launch, no copy node.
    main_case.fill_host_mirror()
    if args.from_hidden:
        def e2e_copy():
            main_case.hidden_dev.copy_(main_case.h_hidden, non_blocking=True)
            main_case.launch()
            main_case.h_y.copy_(main_case.y, non_blocking=True)
        e2e_mapped = None
        h2d = int(main_case.h_hidden.numel() * 2)
    else:
        def e2e_copy():
            buf.inputs.copy_(h_in, non_blocking=True)
            main_case.launch()
            main_case.h_y.copy_(main_case.y, non_blocking=True)

        def e2e_mapped():
            main_case.launch(y=main_case.h_y, host_inputs=h_in)
        h2d = int(h_in.numel())
    es_copy = timed(e2e_copy, None, args.steps, 3, 'timed_e2e_copy')
    es_map = timed(e2e_mapped, None, args.steps, 3, 'timed_e2e_mapped') if e2e_mapped is not None and main_case.T else None
    check_status('e2e region')
    y_mapped_ok = None
    if es_map is not None:
        main_case.write_inputs()
        main_case.launch()
        torch.cuda.synchronize()
        y_mapped_ok = bool(torch.equal(main_case.h_y, main_case.y.cpu()))

    mean_us, med_us = sum(ks) / len(ks), statistics.median(ks)
    e2e_copy_us = sum(es_copy) / len(es_copy)
    e2e_map_us = sum(es_map) / len(es_map) if es_map else None
    mean_us, med_us, span_us, window_us, e2e_copy_us, e2e_map_us = reduce_max([mean_us, med_us, span_us, window_us, e2e_copy_us, e2e_map_us])

    ss_ev = ss_span = None
    if not args.from_hidden:
        ss_ev, ss_span = steady_state(main_case)
        check_status('steady-state region')
        ss_ev, ss_span = reduce_max([ss_ev, ss_span])

    par = None if args.no_parity else parity(main_case)

    sweep = None
    if not args.no_sweep and not args.from_hidden and world > 1 and not args.active_ranks and args.tokens_per_rank == 1:
        sweep = {}
        for name, tokens in sweep_cases(n).items():
            if tokens == main_tokens:                      # the benchmarked case itself: reuse its numbers
                case, ev_mean, sp, win, pr = main_case, mean_us, span_us, window_us, par
            else:
                case = Case(tokens)
                case.write_inputs()
                ev = timed(case.launch, case.write_inputs, 30, 3, 'sweep_' + name)
                sp, win, _ = device_spans(case, reps=8)
                check_status('sweep ' + name)
                ev_mean, sp, win = reduce_max([sum(ev) / len(ev), sp, win])
                pr = parity(case) if not args.no_parity else None
            a_max = max(case.active)
            alg = a_max * W.weight_bytes_per_expert(HIDDEN, INTER, fmt)
            sweep[name] = {'tokens_per_rank': tokens, 'event_us': ev_mean, 'span_us': sp, 'weight_stream_window_us': win,
                           'active_experts_max': a_max, 'algorithmic_bytes': alg,
                           'frac_of_hbm_roofline_events': alg / (ev_mean * 1e-6) / 1e9 / peaks()[0],
                           'frac_of_hbm_roofline_span': alg / (sp * 1e-6) / 1e9 / peaks()[0],
                           'parity_ok': None if pr is None else pr['ok'],
                           'rel_rmse': None if pr is None else pr['rel_rmse_max_over_ranks']}

    # one rank: larger batches (16 .. 128 tokens, forced-balanced over the 48 experts: every expert active, up to 22 rows
    # per expert), on a buffer of their own sized for 128 tokens; same timing recipe, each case checked against the oracle
    tokens_sweep = None
    if not args.no_sweep and not args.from_hidden and world == 1 and args.tokens_per_rank == 1:
        tokens_sweep = {}
        saved = (buf, h_in, h_views)
        buf = mm.get_symm_buffer_for_mega_moe(group, num_experts, 128, TOPK, HIDDEN, INTER, act_format=fmt, num_sms=args.num_sms)
        h_in, h_views = buf.host_inputs()
        try:
            for t in (16, 32, 64, 128):
                case = Case([t])
                case.write_inputs()
                ev = timed(case.launch, case.write_inputs, 30, 3, f'tokens_{t}')
                sp, win, _ = device_spans(case, reps=8)
                check_status(f'tokens sweep {t}')
                pr = parity(case) if not args.no_parity else None
                alg = max(case.active) * W.weight_bytes_per_expert(HIDDEN, INTER, fmt)
                ev_mean = sum(ev) / len(ev)
                tokens_sweep[f'T{t}'] = {'tokens': t, 'rows': t * TOPK, 'event_us': ev_mean, 'span_us': sp, 'active_experts': max(case.active),
                                         'token_tile_rows': buf.tile_image_rows(),
                                         'frac_of_hbm_roofline_events': alg / (ev_mean * 1e-6) / 1e9 / peaks()[0],
                                         'frac_of_hbm_roofline_span': alg / (sp * 1e-6) / 1e9 / peaks()[0],
                                         'parity_ok': None if pr is None else pr['ok'],
                                         'rel_rmse': None if pr is None else pr['rel_rmse_max_over_ranks']}
                if pr is not None and not pr['ok']:
                    par = dict(par or {}, ok=False, failed_case=f'tokens sweep T{t}')
        finally:
            buf, h_in, h_views = saved

    fail = par is not None and not par['ok']
    if rank == 0:
        peak, peak_src = peaks()
        a_max = max(main_case.active)
        alg_bytes = a_max * W.weight_bytes_per_expert(HIDDEN, INTER, fmt)
        achieved = alg_bytes / (mean_us * 1e-6) / 1e9 if alg_bytes else 0.0
        hbm_us = alg_bytes / (peak * 1e9) * 1e6
        nvl_b = nvlink_bytes(main_case)
        nvl_us = (nvl_b / (NVLINK_GBS * 1e9) * 1e6 + NVLINK_RTT_US) if world > 1 else 0.0
        roof_us = max(hbm_us, nvl_us)
        ratio, traffic_src = recorded_traffic(fmt, n)
        e2e_us, e2e_mode = e2e_copy_us, 'one pinned host-to-device copy of the input region + launch + device-to-host copy of y'
        if e2e_map_us is not None and y_mapped_ok and e2e_map_us < e2e_copy_us:
            e2e_us, e2e_mode = e2e_map_us, 'one launch: the kernel reads the inputs from pinned host memory and writes y to pinned host memory'
        roofline = {'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
                    'traffic': int(alg_bytes * ratio) if ratio else None, 'peak_source': peak_src,
                    'algorithmic_bytes_per_launch': alg_bytes, 'active_experts_per_rank': main_case.active,
                    'frac_device_span': alg_bytes / (span_us * 1e-6) / 1e9 / peak if alg_bytes else 0.0,
                    'weight_stream': None if not window_us else {
                        'window_us': window_us, 'gbs': alg_bytes / (window_us * 1e-6) / 1e9,
                        'frac_of_measured_peak': alg_bytes / (window_us * 1e-6) / 1e9 / peak,
                        'frac_of_8000_gbs': alg_bytes / (window_us * 1e-6) / 1e9 / 8000.0,
                        'definition': 'algorithmic bytes / (first weight request of any SM -> last streamed unit in shared memory), max over ranks'},
                    'time_roofline_us': {'hbm': hbm_us, 'nvlink': nvl_us, 'max': roof_us, 'nvlink_bytes_sent_per_rank': nvl_b,
                                         'nvlink_gbs': NVLINK_GBS, 'nvlink_rtt_us': NVLINK_RTT_US if world > 1 else 0.0,
                                         'frac_events': roof_us / mean_us, 'frac_device_span': roof_us / span_us}}
        if traffic_src:
            roofline['traffic_source'] = traffic_src
        line = {'metric': 'moe_layer_kernel_us', 'value': mean_us, 'unit': 'us', 'n_gpus': n, 'steps': args.steps,
                'warmup': W_WARM, 'ms_per_step': mean_us / 1e3, 'higher_is_better': False, 'scaling': 'weak',
                'vs_baseline': None, 'dtype': DTYPE_NAME[fmt], 'data': 'synthetic',
                'config': workload_config(args, n, main_tokens),
                'timing': 'CUDA events around each launch, mean of the timed steps, max over ranks',
                'median_us': med_us, 'device_span_us_median': span_us,
                'device_span_definition': 'first instruction of the earliest SM to the exit of the last SM (globaltimer), median of 10 launches, max over ranks',
                'phases_us_last_launch_rank0': phases, 'sm_phases_us_rank0_min_median_max': sm_summary, 'wall_s': t_wall,
                'event_floor_us': {'nothing_between_events': statistics.median(floor), 'one_element_kernel': statistics.median(floor_k)},
                'steady_state_no_flush': None if ss_ev is None else {
                    'event_us': ss_ev, 'device_span_us': ss_span,
                    'what': 'no L2 flush between steps, routed experts rotate over six disjoint groups (300 MB of weights per rank, '
                            'more than the L2 holds): the weights still come from HBM, the kernel code stays cached'},
                'clocks': clocks, 'gpu_launches': args.steps,
                'tuning': {k: mm._lib.load().mm_get_tuning(v) for k, v in mm._lib.TUNE.items()},
                'e2e': {'value': e2e_us, 'unit': 'us', 'mode': e2e_mode, 'h2d_bytes_per_step': h2d,
                        'd2h_bytes_per_step': int(main_case.h_y.numel() * 2), 'with_copies_us': e2e_copy_us,
                        'mapped_host_memory_us': e2e_map_us, 'mapped_output_equals_device_output': y_mapped_ok},
                'roofline': roofline, 'parity': par}
        if sweep is not None:
            line['m_sweep'] = sweep
        if tokens_sweep is not None:
            line['tokens_sweep'] = tokens_sweep
        if not args.no_cpu_baseline and n == 1:
            us, us_pre, cores = cpu_reference_us(main_tokens[0], fmt, 5)
            line['cpu_baseline'] = {'value': us, 'unit': 'us', 'cores': cores, 'kind': 'port',
                                    'value_weights_predequantised': us_pre,
                                    'sample': f'5 repetitions (after 1 warm-up) of the same layer ({main_tokens[0]} token(s) x top-8 over 48 '
                                              'experts) in the pure-torch oracle; value: weights dequantised inside the timed '
                                              'call, value_weights_predequantised: dequantised once beforehand'}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if fail:
        sys.exit(3)


if __name__ == '__main__':
    main()
