"""Benchmark of the fused MegaMoE layer: kernel microseconds per layer (max over ranks) and HBM roofline fraction.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--tokens-per-rank T] [--format mxfp4|nvfp4]

N = 1 runs the single-GPU configuration (48 local experts, the per-rank work of the 8-rank global-M=8 case: 8 routed
rows on 8 experts). Under torchrun (N > 1) every rank owns 48 experts and feeds T tokens (default 1), i.e. the
8-rank run is the reference's headline case E=384 / H=3072 / I=1280 / top-8 / global M=8. One JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, TOPK, E_LOCAL = 3072, 1280, 8, 48
DTYPE_NAME = {'mxfp4': 'fp4 (e2m1) x fp4, fp32 accumulate', 'nvfp4': 'fp4 (e2m1) x fp4, fp32 accumulate',
              'fp8': 'fp8 (e4m3) x fp4 (e2m1), fp32 accumulate'}
PUBLISHED_US = {}          # BASELINE.json `published` is empty: no number measured for this exact metric


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured (MEASURED_PEAKS.json)'
    return 6650.0, 'fallback'


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
    """The reference's pure-torch quantised MoE (the CPU oracle port) on the host cores: microseconds per layer."""
    import torch
    from oracle import megamoe_oracle as O
    from tests import util_moe as U
    if threads:
        torch.set_num_threads(threads)
    w, gs1, gs2 = O.make_expert_weights(E_LOCAL, HIDDEN, INTER, fmt, seed=0, std=0.02)
    idx, tw = O.balanced_routing(tokens, 0, 1, E_LOCAL, TOPK)
    _, inp, _ = U.make_rank_inputs(tokens, HIDDEN, fmt, 1, idx, tw)
    times = []
    for i in range(reps + 1):
        t0 = time.perf_counter()
        O.moe_layer_reference([inp], [w], fmt, E_LOCAL, clamp=10.0, w1_global_scale=gs1, w2_global_scale=gs2)
        if i:
            times.append((time.perf_counter() - t0) * 1e6)
    return statistics.median(times), torch.get_num_threads()


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    us, cores = cpu_reference_us(args.tokens_per_rank, args.format, max(args.steps, 3))
    sample = (f'{max(args.steps, 3)} repetitions (after 1 warm-up) of one rank\'s layer: {args.tokens_per_rank} token(s) x top-8 '
              f'over 48 experts, H=3072, I=1280, {args.format}; weights dequantised inside the timed call')
    line = {'impl': 'reference', 'metric': 'moe_layer_kernel_us', 'value': us, 'unit': 'us', 'n_gpus': args.gpus,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': us / 1e3, 'higher_is_better': False,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': DTYPE_NAME[args.format], 'data': 'synthetic',
            'config': workload_config(args, args.gpus),
            'cpu_baseline': {'value': us, 'unit': 'us', 'cores': cores, 'kind': 'port', 'sample': sample},
            'e2e': {'value': us, 'unit': 'us', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}
    print(json.dumps(line))


def workload_config(args, n):
    return {'workload': f'EP{n} {"W4A8 (MXFP4 x FP8)" if args.format == "fp8" else "W4A4 " + args.format.upper()} MegaMoE layer, E={E_LOCAL * n} ({E_LOCAL}/rank), H={HIDDEN}, '
                        f'I={INTER}, top-{TOPK}, {"router-picked" if getattr(args, "from_hidden", False) else "forced-balanced"} routing, {args.tokens_per_rank} token(s) per rank '
                        f'(global M={args.tokens_per_rank * n}), weights ~N(0,0.02)'
                        + (', from bf16 hidden states: router GEMM, top-8 and token quantisation fused into the same kernel (routing as the router picks it)' if getattr(args, 'from_hidden', False) else ''),
            'l2': 'flushed by a 256 MiB write before every timed step; then the inputs are copied into the buffer views', 'parallelism': f'ep{n}'}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--tokens-per-rank', type=int, default=1)
    ap.add_argument('--format', default='mxfp4', choices=['mxfp4', 'nvfp4', 'fp8'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--num-sms', type=int, default=0)
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
    n, fmt, T = world, args.format, args.tokens_per_rank
    num_experts = E_LOCAL * n
    W_WARM = max(args.warmup, 3)

    buf = mm.get_symm_buffer_for_mega_moe(group, num_experts, max(T, 16), TOPK, HIDDEN, INTER, act_format=fmt,
                                          num_sms=args.num_sms)
    l1, l2, (gs1, gs2) = W.make_layer_weights(E_LOCAL, HIDDEN, INTER, fmt, seed=1000 + rank)
    x_gs, mid_gs = (1.0 / 64.0, 1.0 / 512.0) if fmt == 'nvfp4' else (1.0, 1.0)
    _, xq, xsf = W.make_tokens(T, HIDDEN, fmt, seed=2000 + rank, global_scale=x_gs)
    idx, tw = W.balanced_routing(T, rank, n, num_experts, TOPK, device='cuda')
    all_idx = [W.balanced_routing(T, r, n, num_experts, TOPK)[0] for r in range(n)]
    active = W.active_experts_per_rank(all_idx, num_experts, n)
    y = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device='cuda')
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device='cuda')
    align = torch.ones(1, device='cuda')
    # pinned host copies for the end-to-end leg
    h_x, h_sf = xq.cpu().pin_memory(), xsf.cpu().pin_memory()
    h_idx, h_w = idx.cpu().pin_memory(), tw.cpu().pin_memory()
    h_y = torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory()

    def write_inputs_from_device():
        if T:
            buf.x[:T].copy_(xq); buf.x_sf[:T].copy_(xsf); buf.topk_idx[:T].copy_(idx); buf.topk_weights[:T].copy_(tw)

    def launch():
        if fmt == 'fp8':
            mm.fp8_fp4_mega_moe(y, l1, l2, buf, activation_clamp=10.0, fast_math=True)
        else:
            mm.fp4_fp4_mega_moe(y, l1, l2, buf, activation_clamp=10.0, fast_math=True, x_global_scale=x_gs,
                                l1_global_scale=gs1, l2_global_scale=gs2, mid_global_scale=mid_gs)

    if args.from_hidden:
        # router over all experts (the same weights on every rank), hidden states ~ N(0, 1); the routing is whatever the
        # router picks (top-8 of softmax), so the active experts per rank are counted from the receive statistics
        g = torch.Generator(device='cuda').manual_seed(77)
        wr = (torch.randn((num_experts, HIDDEN), generator=g, device='cuda') / HIDDEN ** 0.5).to(torch.bfloat16)
        g = torch.Generator(device='cuda').manual_seed(3000 + rank)
        hidden_src = torch.randn((T, HIDDEN), generator=g, device='cuda').to(torch.bfloat16)
        hidden_dev = hidden_src.clone()
        h_hidden = hidden_src.cpu().pin_memory()
        ws = torch.zeros(mm.fe_workspace_bytes(buf), dtype=torch.uint8, device='cuda')
        stats = torch.zeros(E_LOCAL, dtype=torch.int32, device='cuda')

        def write_inputs_from_device():                 # noqa: F811
            hidden_dev.copy_(hidden_src)

        def launch(stats_arg=None):                     # noqa: F811
            mm.mega_moe_from_hidden(y, hidden_dev, wr, l1, l2, buf, ws, cumulative_local_expert_recv_stats=stats_arg,
                                    activation_clamp=10.0, fast_math=True, x_global_scale=x_gs, l1_global_scale=gs1,
                                    l2_global_scale=gs2, mid_global_scale=mid_gs)
        if world > 1:
            dist.barrier()
        launch(stats)
        torch.cuda.synchronize()
        mine = torch.tensor([int((stats > 0).sum())], device='cuda')
        if world > 1:
            gathered = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            active = [int(v) for v in gathered]
        else:
            active = [int(mine)]

    def timed(step_fn, steps, warm, e2e=False):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for _ in range(20):                        # let the host run ahead of the GPU: events then bracket the kernel,
            flush.zero_()                          # not the host's launch latency
        for i in range(warm + steps):
            if i == warm:
                torch.cuda.nvtx.range_push('timed_e2e' if e2e else 'timed')
            flush.zero_()
            if not e2e:
                write_inputs_from_device()         # flush -> input copy -> rank alignment -> kernel, as the reference's
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

    write_inputs_from_device()
    sampler = ClockSampler(local)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    t_wall0 = time.perf_counter()
    ks = timed(launch, args.steps, W_WARM)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall0
    clocks = sampler.stop() if rank == 0 else None
    # device-side span (first SM's entry stamp to the last SM's exit stamp, globaltimer) of a few extra launches
    spans = []
    for _ in range(10):
        flush.zero_()
        write_inputs_from_device()
        if world > 1:
            dist.all_reduce(align)
        launch()
        stamps = buf.phase_stamps()
        spans.append((stamps[8] - stamps[0]) / 1e3)
    span_us = statistics.median(spans)
    phase_names = ['entry', 'dispatched', 'dispatch_headers_seen', 'scheduled', 'tasks_done', None, None, 'exit', 'last_sm_exit',
                   'frontend_done', 'last_sm_tasks_done', 'last_sm_scheduled']
    phases = {n: round((stamps[i] - stamps[0]) / 1e3, 2) for i, n in enumerate(phase_names) if n and stamps[i]}
    st, words = buf.device_status()
    if st != 0:
        raise RuntimeError(f'device status {st}: {[hex(v) for v in words[:4]]}')

    # end-to-end leg: the step's inputs sit in one pinned host mirror of the buffer's input region (filled once here, as a
    # serving loop would fill it per step) and reach the device with a single copy; y comes back to pinned memory
    h_in, h_views = buf.host_inputs()
    if T:
        h_views['x'][:T].copy_(h_x); h_views['x_sf'][:T].copy_(h_sf)
        h_views['topk_idx'][:T].copy_(h_idx); h_views['topk_weights'][:T].copy_(h_w)

    def e2e_step():
        buf.inputs.copy_(h_in, non_blocking=True)
        launch()
        h_y.copy_(y, non_blocking=True)
    if args.from_hidden:
        def e2e_step():                                 # noqa: F811  (hidden states are the step's only input)
            hidden_dev.copy_(h_hidden, non_blocking=True)
            launch()
            h_y.copy_(y, non_blocking=True)
    es = timed(e2e_step, args.steps, 3, e2e=True)

    mean_us, e2e_us = sum(ks) / len(ks), sum(es) / len(es)
    t = torch.tensor([mean_us, e2e_us, statistics.median(ks), span_us], device='cuda', dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mean_us, e2e_us, med_us, span_us = t.tolist()
    if rank == 0:
        peak, peak_src = peaks()
        a_max = max(active)
        alg_bytes = a_max * W.weight_bytes_per_expert(HIDDEN, INTER, fmt)
        achieved = alg_bytes / (mean_us * 1e-6) / 1e9
        line = {'metric': 'moe_layer_kernel_us', 'value': mean_us, 'unit': 'us', 'n_gpus': n, 'steps': args.steps,
                'warmup': W_WARM, 'ms_per_step': mean_us / 1e3, 'higher_is_better': False, 'scaling': 'weak',
                'vs_baseline': None, 'dtype': DTYPE_NAME[fmt], 'data': 'synthetic',
                'config': workload_config(args, n), 'timing': 'CUDA events around each launch, mean of the timed steps, max over ranks',
                'median_us': med_us, 'device_span_us_median': span_us, 'phases_us_sm0_last_launch': phases, 'wall_s': t_wall,
                'clocks': clocks, 'gpu_launches': args.steps,
                'e2e': {'value': e2e_us, 'unit': 'us',
                        'h2d_bytes_per_step': int(h_hidden.numel() * 2 if args.from_hidden else h_in.numel()),
                        'd2h_bytes_per_step': int(h_y.numel() * 2)},
                'roofline': {'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
                             'traffic': (int(alg_bytes * 1.0023) if (fmt == 'mxfp4' and n == 1) else None), 'traffic_source': 'dram__bytes_read+write of one ncu capture of this workload, scaled by the active experts (profiles/)', 'peak_source': peak_src,
                             'algorithmic_bytes_per_launch': alg_bytes, 'active_experts_per_rank': active}}
        if not args.no_cpu_baseline and n == 1:
            us, cores = cpu_reference_us(T, fmt, 5)
            line['cpu_baseline'] = {'value': us, 'unit': 'us', 'cores': cores, 'kind': 'port',
                                    'sample': f'5 repetitions (after 1 warm-up) of the same layer ({T} token(s) x top-8 over 48 '
                                              'experts) in the pure-torch oracle, weights dequantised inside the timed call'}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
