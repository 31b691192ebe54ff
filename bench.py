"""Benchmark of the quantization hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows R] [--no-ops]

Workload ("cfg5"): per-token FP8 e4m3 cast, groups of 128, power-of-two scales packed as ue8m0 in the
column-major layout, of a bf16 [262144, 7168] tensor ~ N(0,1) with 0.1% x100 outliers, token dimension
split evenly over the N ranks (no collective on the data path).  One step = one cast of the rank's shard.

  value     Mtokens/s over all ranks, inputs resident in HBM, device-timed (CUDA events), max over ranks
  e2e       the same cast through tilekernels_b200.host.per_token_cast_host: pinned host input ->
            device -> cast -> pinned host outputs, all copies inside the timed region
  roofline  algorithmic bytes (input + output + scales, each once) / kernel time against the measured
            HBM copy bandwidth of this pool (MEASURED_PEAKS.json, else the documented fallback)
  ops       (N = 1) the other benchmark workloads, each timed L2-cold by rotating over buffer sets
            larger than twice the L2
  cpu_baseline  the CPU oracle (a C/OpenMP port of the reference's PyTorch path) on a bounded row sample

--impl reference times that CPU port alone, on all host cores, as the reference arm.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOTAL_ROWS = 262144
HIDDEN = 7168
GROUP = 128
L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only without MEASURED_PEAKS.json
# DRAM bytes per token of the dominant kernel from the ncu capture summarised in
# profiles/per_token_cast_e4m3_ue8m0_cfg5.md: (dram__bytes_read.sum + dram__bytes_write.sum) of one launch
# over 32768 rows / 32768.  Traffic is proportional to the row count, so a launch's traffic is this x rows.
NCU_DRAM_BYTES_PER_TOKEN = 20465


def bytes_per_token() -> int:
    """Algorithmic bytes per token of the cfg5 cast: bf16 in, e4m3 out, one ue8m0 byte per 128 values."""
    return HIDDEN * 2 + HIDDEN + HIDDEN // GROUP


def hbm_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return FALLBACK_HBM_GBS, 'fallback'


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only queries) from a background
    thread every few milliseconds while the timed region runs."""

    REASONS = {0x8: 'hw_slowdown', 0x40: 'hw_thermal_slowdown', 0x20: 'sw_thermal_slowdown', 0x4: 'sw_power_cap'}

    def __init__(self, torch, device_index: int, period_s: float = 0.002):
        self.period = period_s
        self.samples = []  # (time, sm_mhz, reasons_mask, power_w)
        self.handle = None
        self.stop_flag = threading.Event()
        try:
            import pynvml
            self.nvml = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith('GPU-'):
                uuid = 'GPU-' + uuid
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.handle = None
            self.max_sm = None

    def _loop(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                power = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((time.perf_counter(), sm, mask, power))
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        if self.handle is not None:
            self.thread.join(timeout=2)

    def summary(self, t0: float = None, t1: float = None) -> dict:
        """Median SM clock and the set of throttle reasons seen between host times t0 and t1 (all samples if None)."""
        rows = [r for r in self.samples if (t0 is None or r[0] >= t0) and (t1 is None or r[0] <= t1)]
        reasons = set()
        for _, _, mask, _ in rows:
            for bit, name in self.REASONS.items():
                if mask & bit:
                    reasons.add(name)
        return {'sm_mhz': statistics.median(r[1] for r in rows) if rows else None, 'sm_max_mhz': self.max_sm,
                'reasons': sorted(reasons), 'samples': len(rows),
                'power_w_max': round(max(r[3] for r in rows), 1) if rows else None}


def time_steps(torch, fn, steps: int, warmup: int, barrier):
    """Milliseconds for `steps` calls of fn on the current stream, after `warmup` calls; barrier + sync on both
    sides.  Also returns the host times that bracket the timed region (for the clock samples)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    return start.elapsed_time(stop), t0, t1


def time_graph(torch, op, inputs, launches: int, replays: int = 7):
    """Device time per launch (microseconds; median and minimum over replays) of `op` applied to the inputs in
    rotation, with all launches captured in one CUDA graph so that host launch overhead is not measured.
    Every output of a capture stays alive until the capture ends, so outputs rotate through distinct
    addresses like the inputs do."""
    for x in inputs:
        op(x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    keep = []
    with torch.cuda.graph(graph):
        for i in range(launches):
            keep.append(op(inputs[i % len(inputs)]))
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / launches)
    del keep, graph
    return statistics.median(times), min(times)


def bench_other_ops(torch, quant, device, count_bytes) -> list:
    """cfg1-cfg4 on one GPU.  Working sets below the L2 size are timed L2-cold: each launch uses the next of
    `sets` distinct input/output sets whose total size exceeds twice the L2."""
    from tilekernels_b200 import moe
    from tilekernels_b200.testing import make_config_input
    peak, _ = hbm_peak()
    specs = [
        ('cfg1 per_token_cast e4m3 g128 fp32-sf [4096,7168]', 'cfg1', None, lambda x: quant.per_token_cast(x, 'e4m3', 128)),
        ('cfg1 per_token_cast e4m3 g128 round_sf [4096,7168]', 'cfg1', None, lambda x: quant.per_token_cast(x, 'e4m3', 128, round_sf=True)),
        ('cfg2 per_block_cast e4m3 128x128 [7168,2048]', 'cfg2', None, lambda x: quant.per_block_cast(x, 'e4m3', (128, 128))),
        ('cfg2 per_channel_cast e4m3 128 [7168,2048]', 'cfg2', None, lambda x: quant.per_channel_cast(x, 'e4m3', 128)),
        ('cfg3 swiglu_forward_and_per_token_cast e4m3 g128 [16384,4096]', 'cfg3', None,
         lambda x: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128)),
        ('cfg4 per_token_cast e2m1 g32 ue8m0 [32768,7168]', 'cfg4', None,
         lambda x: quant.per_token_cast(x, 'e2m1', 32, None, True, True, True)),
        ('cfg4 per_token_cast e5m6 [32768,7168]', 'cfg4', None, lambda x: quant.per_token_cast(x, 'e5m6', x.shape[1])),
    ]
    ue = dict(use_tma_aligned_col_major_sf=True, round_sf=True, use_packed_ue8m0=True)
    gather = torch.randint(0, 7168, (8192,), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    gather[::11] = -1
    gather = gather.to(device)

    def backward_inputs(x):
        rows, hidden = x.shape[0], x.shape[1] // 2
        g = torch.Generator().manual_seed(11)
        grad_out = torch.randn((rows, hidden), generator=g).to(torch.bfloat16).to(device)
        weight = torch.rand((rows // 8, 8), generator=g).to(device)
        pos = torch.randperm(rows, generator=g).to(torch.int32)
        token_topk_to_pos = torch.empty(rows, dtype=torch.int32)
        token_topk_to_pos[pos.long()] = torch.arange(rows, dtype=torch.int32)
        return (quant.per_token_cast(x, 'e4m3', 128, round_sf=True), grad_out, weight, pos.to(device), token_topk_to_pos.view(-1, 8).to(device))


    def expand_inputs(x):
        q, sf = quant.per_token_cast(x, 'e4m3', 128, None, **ue)
        positions = torch.randperm(x.shape[0] * 8, generator=torch.Generator().manual_seed(13)).to(torch.int32)
        return ((q, sf.contiguous()), positions.view(-1, 8).to(device), torch.zeros(x.shape[0] * 8, dtype=torch.int32, device=device))

    # the rows next to the hot path (dequantisation, re-quantisation, fused / transposing per-channel casts):
    # `prepare` turns the bf16 workload tensor into the op's input
    specs += [
        ('cfg4 per_token_cast_back e4m3 g128 ue8m0 -> bf16 [32768,7168]', 'cfg4', lambda x: quant.per_token_cast(x, 'e4m3', 128, None, **ue),
         lambda q: (quant.per_token_cast_back(q, 'bf16', 128),)),
        ('cfg4 per_token_cast_back e5m6 -> bf16 [32768,7168]', 'cfg4', lambda x: quant.per_token_cast(x, 'e5m6', x.shape[1]),
         lambda q: (quant.per_token_cast_back(q, 'bf16', 7168, x_special_fmt='e5m6'),)),
        ('cfg4 per_token_cast e4m3 g128 of FP8 input with 128x128 ue8m0 scales [32768,7168]', 'cfg4',
         lambda x: quant.per_block_cast(x, 'e4m3', (128, 128), **ue), lambda q: quant.per_token_cast(q, 'e4m3', 128, (128, 128), **ue)),
        ('cfg2 per_channel_cast_fused bf16 + gather of 8192 rows [7168,2048]', 'cfg2', None,
         lambda x: quant.per_channel_cast_fused(x, 'e4m3', 128, False, None, gather)),
        ('cfg2 per_channel_cast_and_transpose 128 [7168,2048]', 'cfg2', None, lambda x: quant.per_channel_cast_and_transpose(x, 'e4m3', 128)),
        ('cfg3 swiglu_backward_and_per_token_cast g128 round_sf, input scales powers of two [16384,4096]', 'cfg3',
         backward_inputs, lambda a: quant.swiglu_backward_and_per_token_cast(*a, 128, True)),
        ('cfg1 moe.expand_to_fused_with_sf of the FP8 cast, 8 positions per token, ue8m0 scales [4096,7168] -> [32768,7168]', 'cfg1',
         expand_inputs, lambda a: moe.expand_to_fused_with_sf(a[0], 128, a[1], a[2], True)),
    ]

    def clone(v):
        return tuple(clone(t) for t in v) if isinstance(v, tuple) else v.clone()

    cache, results = {}, []
    for label, cfg, prepare, op in specs:
        if cfg not in cache:
            cache.clear()
            cache[cfg] = make_config_input(cfg).to(device)
        x = cache[cfg] if prepare is None else prepare(cache[cfg])
        out = op(x)
        nbytes = count_bytes(x, out)
        sets = max(2, -(-2 * L2_BYTES // nbytes) + 1)
        del out
        xs = [x] + [clone(x) for _ in range(sets - 1)]
        med, best = time_graph(torch, op, xs, launches=2 * sets)
        del xs, x
        torch.cuda.empty_cache()
        results.append({'op': label, 'bytes': nbytes, 'us_median': round(med, 2), 'us_min': round(best, 2),
                        'gbs': round(nbytes / med / 1e3, 1), 'frac_of_hbm_peak': round(nbytes / med / 1e3 / peak, 3),
                        'l2': f'cold: {sets} rotating input/output sets, {2 * sets} launches per CUDA graph replay'})
    return results


def cpu_model() -> str:
    """Model name of the host CPU (first entry of /proc/cpuinfo), for the CPU baseline's record."""
    try:
        with open('/proc/cpuinfo') as f:
            for line in f:
                if line.lower().startswith('model name'):
                    return line.split(':', 1)[1].strip()
    except OSError:
        pass
    return 'unknown'


def oracle_rate(rows: int, threads: int, repeats: int = 1) -> float:
    """Mtokens/s of the CPU oracle on `rows` rows of the cfg5 workload (best of `repeats`)."""
    import torch

    import oracle
    from tilekernels_b200.testing import make_config_input
    torch.set_num_threads(threads)
    os.environ.setdefault('OMP_NUM_THREADS', str(threads))
    x = make_config_input('cfg5', rows)
    oracle.cast(x[:256], 'e4m3', (1, GROUP), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    best = float('inf')
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.cast(x, 'e4m3', (1, GROUP), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
        best = min(best, time.perf_counter() - t0)
    return rows / best / 1e6


def run_reference(args) -> None:
    """Reference arm: the CPU port of the reference's PyTorch path on all host cores, bounded sample per step."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    import torch

    import oracle
    from tilekernels_b200.testing import make_config_input
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows = args.rows or 16384
    x = make_config_input('cfg5', rows)
    kw = dict(round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    for _ in range(max(1, min(args.warmup, 3))):
        oracle.cast(x, 'e4m3', (1, GROUP), **kw)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.cast(x, 'e4m3', (1, GROUP), **kw)
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt / 1e6
    sample = f'{rows} of {TOTAL_ROWS} rows per step'
    line = {
        'impl': 'reference', 'metric': 'per_token_cast_fp8_e4m3_g128_ue8m0_throughput', 'value': round(value, 3), 'unit': 'Mtokens/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(dt / args.steps * 1e3, 3),
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': f'cfg5 per-token FP8 e4m3 cast, group 128, ue8m0 col-major scales, bf16 [{TOTAL_ROWS},{HIDDEN}]',
                   'sample': sample},
        'hbm_gbs': round(value * bytes_per_token() / 1e3, 3),
        'cpu_baseline': {'value': round(value, 3), 'unit': 'Mtokens/s', 'cores': cores, 'kind': 'port', 'sample': sample, 'cpu': cpu_model()},
        'e2e': {'value': round(value, 3), 'unit': 'Mtokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from tilekernels_b200 import host, quant
    from tilekernels_b200.sharding import shard_rows
    from tilekernels_b200.testing import count_bytes, make_config_input

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    assert world == args.gpus, f'--gpus {args.gpus} but WORLD_SIZE={world}'
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()

    total_rows = args.rows or TOTAL_ROWS
    first_row, last_row = shard_rows(total_rows, rank, world, alignment=4096)  # whole generator chunks per rank
    rows = last_row - first_row
    assert rows > 0 and rows % 4 == 0, 'every rank needs rows, in multiples of 4'

    # the rank's shard, generated on the host (pinned), then copied once for the device-resident measurement
    x_host = torch.empty((rows, HIDDEN), dtype=torch.bfloat16, pin_memory=True)
    make_config_input('cfg5', rows, first_row=first_row, out=x_host)
    x = x_host.to(device, non_blocking=True)
    torch.cuda.synchronize()

    def step():
        return quant.per_token_cast(x, 'e4m3', GROUP, None, True, True, True)

    with ClockSampler(torch, local_rank) as sampler:
        ms, t0, t1 = time_steps(torch, step, args.steps, args.warmup, barrier)
    clocks = sampler.summary(t0, t1)
    if clocks['samples'] == 0:  # a timed region shorter than the sampling period: use the samples around it
        clocks = sampler.summary()

    # end to end through the host-buffer API
    out_host = torch.empty((rows, HIDDEN), dtype=torch.float8_e4m3fn, pin_memory=True)
    sf_host = torch.empty((HIDDEN // GROUP // 4, rows), dtype=torch.int32, pin_memory=True)
    pipe = host.HostCastPipeline(device, hidden=HIDDEN, max_rows=rows)

    def e2e_step():
        pipe.per_token_cast_host(x_host, 'e4m3', GROUP, out_host, sf_host)

    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e, _, _ = time_steps(torch, e2e_step, e2e_steps, 3, barrier)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()

    if rank == 0:
        peak, peak_kind = hbm_peak()
        ms_per_step = ms / args.steps
        value = total_rows / (ms_per_step * 1e-3) / 1e6
        kernel_gbs = rows * bytes_per_token() / (ms_per_step * 1e-3) / 1e9  # per GPU: one launch per step on each rank
        e2e_value = total_rows / (ms_e2e / e2e_steps * 1e-3) / 1e6
        line = {
            'metric': 'per_token_cast_fp8_e4m3_g128_ue8m0_throughput', 'value': round(value, 2), 'unit': 'Mtokens/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms_per_step, 4),
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'config': {'workload': f'cfg5 per-token FP8 e4m3 cast, group 128, ue8m0 col-major scales, bf16 [{total_rows},{HIDDEN}]',
                       'rows_per_rank': rows, 'sharding': f'token dimension split over {world} rank(s), no collective',
                       'l2': 'inputs larger than L2 (no flush needed)'},
            'hbm_gbs': round(kernel_gbs * world, 1),
            'pct_of_8tbs': round(kernel_gbs / 8000.0 * 100, 1),
            'clocks': clocks,
            # bytes of all ranks together, like `value`
            'e2e': {'value': round(e2e_value, 3), 'unit': 'Mtokens/s', 'h2d_bytes_per_step': total_rows * HIDDEN * 2,
                    'd2h_bytes_per_step': total_rows * HIDDEN + total_rows * (HIDDEN // GROUP), 'steps': e2e_steps,
                    'api': 'tilekernels_b200.host.HostCastPipeline.per_token_cast_host (pinned host buffers)'},
            'gpu_launches': args.steps,
            'roofline': {'bound': 'hbm', 'achieved': round(kernel_gbs, 1), 'peak': peak, 'unit': 'GB/s',
                         'frac': round(kernel_gbs / peak, 4), 'peak_source': f'of {peak_kind}',
                         'traffic': None if NCU_DRAM_BYTES_PER_TOKEN is None else NCU_DRAM_BYTES_PER_TOKEN * rows,
                         'algorithmic_bytes_per_launch': rows * bytes_per_token(), 'kernel': 'group_cast_kernel<bf16,e4m3,LPG=8>'},
        }
        if world == 1:
            cores = os.cpu_count() or 1
            sample_rows = 32768
            line['cpu_baseline'] = {'value': round(oracle_rate(sample_rows, cores, repeats=3), 3), 'unit': 'Mtokens/s', 'cores': cores,
                                    'kind': 'port', 'sample': f'{sample_rows} of {TOTAL_ROWS} rows, best of 3', 'cpu': cpu_model()}
            if not args.no_ops:
                del x
                torch.cuda.empty_cache()
                line['ops'] = bench_other_ops(torch, quant, device, count_bytes)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--rows', type=int, default=0, help='total rows (default 262144); for quick runs')
    ap.add_argument('--no-ops', action='store_true', help='skip the per-op table of the other workloads')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
