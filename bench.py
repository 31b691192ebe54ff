"""Benchmark of the quantization hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows R] [--no-ops] [--records FILE]

Workload ("cfg5"): per-token FP8 e4m3 cast, groups of 128, power-of-two scales packed as ue8m0 in the
column-major layout, of a bf16 [262144, 7168] tensor ~ N(0,1) with 0.1% x100 outliers, token dimension
split evenly over the N ranks (no collective on the data path).  One step = one cast of the rank's shard.

  value     Mtokens/s over all ranks, inputs resident in HBM, device-timed (CUDA events), max over ranks
  e2e       the same cast through tilekernels_b200.host.per_token_cast_host: pinned host input ->
            device -> cast -> pinned host outputs, all copies inside the timed region
  roofline  algorithmic bytes (input + output + scales, each once) / kernel time against the measured
            HBM copy bandwidth of this pool (MEASURED_PEAKS.json, else the documented fallback)
  ops       (N = 1) the other benchmark workloads, each timed L2-cold by rotating over buffer sets
            larger than twice the L2, with a device copy of the same size and the host cost per call beside it;
            --records FILE writes them as JSONL in the record form of the reference's benchmark plugin
  shard_parity  every rank's first and last 4096-row band compared with the CPU checker (outside the timing)
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
TRAFFIC_FILE = os.path.join(ROOT, 'profiles', 'per_token_cast_e4m3_ue8m0_cfg5.traffic.json')


def workload_config(total_rows: int, world: int) -> dict:
    """The `config` object of the JSON line, the same for both arms."""
    return {'workload': f'cfg5 per-token FP8 e4m3 cast, group 128, ue8m0 col-major scales, bf16 [{total_rows},{HIDDEN}]',
            'rows_per_rank': total_rows // world, 'sharding': f'token dimension split over {world} rank(s), no collective',
            'l2': 'inputs larger than L2 (no flush needed)'}


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


def profiled_traffic():
    """DRAM bytes per token of the dominant kernel, from the last profiler capture of it (a small tracked JSON:
    bytes read + written by one launch / its rows, and the commit the capture was taken at).  Traffic is
    proportional to the row count, so a launch's traffic is this x rows.  None if the file is missing."""
    try:
        with open(TRAFFIC_FILE) as f:
            return json.load(f)
    except Exception:
        return None


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


def time_steps(torch, fn, steps: int, warmup: int, barrier, graph_bytes_per_step: int = 0):
    """Milliseconds for `steps` calls of fn on the current stream, after `warmup` calls; barrier + sync on both
    sides.  Also returns the host times that bracket the timed region (for the clock samples) and how the steps
    were launched.

    With graph_bytes_per_step > 0 (the bytes one call allocates) and enough free memory, the `steps` calls are
    captured into ONE CUDA graph after the eager warm-up, replayed once untimed and once timed: a hiccup of the host
    thread then cannot stretch a timed region that is only a few milliseconds long (eight ranks, 0.12 ms per step).
    Results are dropped as they are in an eager loop, so the allocator hands every step the same output memory.
    Otherwise the calls are launched eagerly."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph, mode = None, 'eager calls of the public entry point'
    if graph_bytes_per_step > 0 and 3 * graph_bytes_per_step < torch.cuda.mem_get_info()[0]:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(steps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        mode = 'one CUDA graph of the timed steps, captured from the public entry point after the eager warm-up'
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    if graph is not None:
        graph.replay()
    else:
        for _ in range(steps):
            fn()
    stop.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    ms = start.elapsed_time(stop)
    if graph is not None:
        del graph
        torch.cuda.empty_cache()
    return ms, t0, t1, mode


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


def time_copy(torch, device, nbytes: int) -> float:
    """Microseconds of a device-to-device copy that moves `nbytes` in total (reads nbytes / 2, writes nbytes / 2),
    timed like the ops: CUDA-graph replay over rotating buffer pairs larger than twice the L2.  Two forms are timed
    and the faster one is returned: Tensor.copy_ (the driver's memcpy, which may pick the copy engine) and an
    elementwise kernel over 32-bit words (always on the SMs)."""
    half = max(1024, nbytes // 2 // 1024 * 1024)
    sets = max(2, -(-2 * L2_BYTES // (2 * half)) + 1)
    srcs = [torch.empty(half // 4, dtype=torch.int32, device=device) for _ in range(sets)]
    dsts = [torch.empty(half // 4, dtype=torch.int32, device=device) for _ in range(sets)]
    pairs = list(zip(srcs, dsts))
    memcpy, _ = time_graph(torch, lambda p: p[1].copy_(p[0]), pairs, launches=2 * sets)
    kernel, _ = time_graph(torch, lambda p: torch.bitwise_or(p[0], 0, out=p[1]), pairs, launches=2 * sets)
    return min(memcpy, kernel)


def host_us_per_call(torch, op, x, calls: int = 1000) -> float:
    """Wall-clock microseconds of one eager call of the Python entry point (asserts, output allocation, ctypes,
    launch) on an input so small that the kernel itself does not matter."""
    for _ in range(20):
        op(x)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(calls):
        op(x)
    t1 = time.perf_counter()
    torch.cuda.synchronize()
    return (t1 - t0) / calls * 1e6


def op_specs(torch, quant, moe, device) -> list:
    """The per-op table: the benchmark workloads cfg1-cfg4, the steady-state shapes of the tile kernels and the rows
    next to the hot path.  Each spec: kernel / operation / params (the record fields of the reference's benchmark
    plugin, tests/pytest_benchmark_plugin.py:358-425), the workload tensor it starts from, an optional `prepare`
    (workload tensor -> op input) and the op."""
    ue = dict(use_tma_aligned_col_major_sf=True, round_sf=True, use_packed_ue8m0=True)
    gather = torch.randint(0, 7168, (8192,), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    gather[::11] = -1
    # row indices for the full workload and for the 128-row input of the host-cost measurement
    gathers = {7168: gather.to(device), 128: torch.where(gather < 0, gather, gather % 128).to(device)}

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

    def spec(kernel, operation, cfg, op, prepare=None, **params):
        return {'kernel': kernel, 'operation': operation, 'cfg': cfg, 'op': op, 'prepare': prepare, 'params': params}

    return [
        spec('per_token_cast', 'cfg1', 'cfg1', lambda x: quant.per_token_cast(x, 'e4m3', 128), fmt='e4m3', group=128, sf='fp32'),
        spec('per_token_cast', 'cfg1', 'cfg1', lambda x: quant.per_token_cast(x, 'e4m3', 128, round_sf=True), fmt='e4m3', group=128, sf='fp32 pow2'),
        spec('per_block_cast', 'cfg2', 'cfg2', lambda x: quant.per_block_cast(x, 'e4m3', (128, 128)), fmt='e4m3', block='128x128'),
        spec('per_channel_cast', 'cfg2', 'cfg2', lambda x: quant.per_channel_cast(x, 'e4m3', 128), fmt='e4m3', block='128x1'),
        spec('swiglu_forward_and_per_token_cast', 'cfg3', 'cfg3', lambda x: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128),
             fmt='e4m3', group=128, sf='fp32'),
        spec('swiglu_forward_and_per_token_cast', 'cfg3', 'cfg3', lambda x: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128, **ue),
             fmt='e4m3', group=128, sf='ue8m0'),
        spec('per_token_cast', 'cfg4', 'cfg4', lambda x: quant.per_token_cast(x, 'e2m1', 32, None, True, True, True), fmt='e2m1', group=32, sf='ue8m0'),
        spec('per_token_cast', 'cfg4', 'cfg4', lambda x: quant.per_token_cast(x, 'e5m6', x.shape[1]), fmt='e5m6', group=7168, sf='fp32'),
        # the tile kernels in steady state: 14336 tiles, 16 times the resident blocks
        spec('per_block_cast', 'large', 'cfg4', lambda x: quant.per_block_cast(x, 'e4m3', (128, 128)), fmt='e4m3', block='128x128'),
        spec('per_channel_cast', 'large', 'cfg4', lambda x: quant.per_channel_cast(x, 'e4m3', 128), fmt='e4m3', block='128x1'),
        # the rows next to the hot path
        spec('per_token_cast_back', 'cfg4', 'cfg4', lambda q: (quant.per_token_cast_back(q, 'bf16', 128),),
             lambda x: quant.per_token_cast(x, 'e4m3', 128, None, **ue), fmt='e4m3', group=128, sf='ue8m0', out='bf16'),
        spec('per_token_cast_back', 'cfg4', 'cfg4', lambda q: (quant.per_token_cast_back(q, 'bf16', 7168, x_special_fmt='e5m6'),),
             lambda x: quant.per_token_cast(x, 'e5m6', x.shape[1]), fmt='e5m6', out='bf16'),
        spec('per_token_cast', 'cfg4 requantise', 'cfg4', lambda q: quant.per_token_cast(q, 'e4m3', 128, (128, 128), **ue),
             lambda x: quant.per_block_cast(x, 'e4m3', (128, 128), **ue), fmt='e4m3', group=128, x='e4m3 128x128 ue8m0'),
        spec('per_token_cast', 'cfg4 requantise, fp32 scales', 'cfg4', lambda q: quant.per_token_cast(q, 'e4m3', 128, (1, 128)),
             lambda x: quant.per_token_cast(x, 'e4m3', 128), fmt='e4m3', group=128, x='e4m3 1x128 fp32 scales'),
        spec('per_token_cast', 'cfg4 requantise, FP4 input', 'cfg4', lambda q: quant.per_token_cast(q, 'e4m3', 128, (1, 32), **ue),
             lambda x: quant.per_token_cast(x, 'e2m1', 32, None, **ue), fmt='e4m3', group=128, x='e2m1 1x32 ue8m0'),
        spec('per_channel_cast_fused', 'cfg4 FP8 input', 'cfg4', lambda q: quant.per_channel_cast_fused(q, 'e4m3', 128, False, 128),
             lambda x: quant.per_token_cast(x, 'e4m3', 128), fmt='e4m3', x='e4m3 1x128 fp32 scales'),
        spec('per_channel_cast_fused', 'cfg2 gather', 'cfg2', lambda x: quant.per_channel_cast_fused(x, 'e4m3', 128, False, None, gathers[x.shape[0]]),
             fmt='e4m3', rows_out=8192),
        spec('per_channel_cast_and_transpose', 'cfg2', 'cfg2', lambda x: quant.per_channel_cast_and_transpose(x, 'e4m3', 128), fmt='e4m3', block='128x1'),
        spec('swiglu_forward_and_per_channel_cast_and_transpose', 'cfg3', 'cfg3',
             lambda x: quant.swiglu_forward_and_per_channel_cast_and_transpose(x, 'e4m3', 128), fmt='e4m3', block='128x1'),
        spec('per_block_cast_lossless', 'cfg4', 'cfg4', lambda q: quant.per_block_cast_lossless(q, 'e4m3', (1, 32), (128, 128), True, True, True),
             lambda x: quant.per_token_cast(x, 'e2m1', 32, None, True, True, True), x='e2m1 1x32 ue8m0', fmt='e4m3', block='128x128', sf='ue8m0'),
        spec('swiglu_backward_and_per_token_cast', 'cfg3', 'cfg3', lambda a: quant.swiglu_backward_and_per_token_cast(*a, 128, True),
             backward_inputs, group=128, sf='fp32 pow2', x_sf='pow2'),
        spec('expand_to_fused_with_sf', 'cfg1', 'cfg1', lambda a: moe.expand_to_fused_with_sf(a[0], 128, a[1], a[2], True), expand_inputs,
             x='e4m3 + ue8m0', positions_per_token=8),
    ]


def bench_other_ops(torch, quant, device, count_bytes) -> list:
    """The per-op table on one GPU.  Working sets below the L2 size are timed L2-cold: each launch uses the next of
    `sets` distinct input/output sets whose total size exceeds twice the L2.  Beside every op: a device copy of the
    same number of bytes timed the same way, and the host cost of one eager call."""
    from tilekernels_b200 import moe
    from tilekernels_b200.testing import make_config_input
    peak, _ = hbm_peak()

    def clone(v):
        return tuple(clone(t) for t in v) if isinstance(v, tuple) else v.clone()

    def shape_of(v):
        while isinstance(v, tuple):
            v = v[0]
        return list(v.shape)

    cache, copies, results = {}, {}, []
    for s in op_specs(torch, quant, moe, device):
        cfg, prepare, op = s['cfg'], s['prepare'], s['op']
        if cfg not in cache:
            cache.clear()
            torch.cuda.empty_cache()
            cache[cfg] = make_config_input(cfg).to(device)
        tiny = make_config_input(cfg, 128).to(device)
        host_us = host_us_per_call(torch, op, tiny if prepare is None else prepare(tiny))
        x = cache[cfg] if prepare is None else prepare(cache[cfg])
        out = op(x)
        nbytes = count_bytes(x, out)
        sets = max(2, -(-2 * L2_BYTES // nbytes) + 1)
        del out
        xs = [x] + [clone(x) for _ in range(sets - 1)]
        med, best = time_graph(torch, op, xs, launches=2 * sets)
        shape = shape_of(x)
        del xs, x
        torch.cuda.empty_cache()
        if nbytes not in copies:
            copies[nbytes] = time_copy(torch, device, nbytes)
            torch.cuda.empty_cache()
        params = dict(s['params'], shape=shape)
        results.append({'kernel': s['kernel'], 'operation': s['operation'], 'params': params, 'bytes': nbytes,
                        'time_us': round(med, 2), 'us_min': round(best, 2), 'bandwidth_gbs': round(nbytes / med / 1e3, 1),
                        'frac_of_hbm_peak': round(nbytes / med / 1e3 / peak, 3),
                        'copy_us': round(copies[nbytes], 2), 'frac_of_same_size_copy': round(copies[nbytes] / med, 3),
                        'host_us_per_call': round(host_us, 1),
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
        'config': workload_config(TOTAL_ROWS, args.gpus),
        'hbm_gbs': round(value * bytes_per_token() / 1e3, 3),
        'cpu_baseline': {'value': round(value, 3), 'unit': 'Mtokens/s', 'cores': cores, 'kind': 'port', 'sample': sample, 'cpu': cpu_model()},
        'e2e': {'value': round(value, 3), 'unit': 'Mtokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


def shard_parity(torch, oracle, x_host, out, sf, rows: int) -> bool:
    """Outside every timed region: the first and the last 4096-row band of this rank's shard, cast by the oracle on
    the host, must equal what the rank's kernel wrote (codes and scale words)."""
    ok = True
    band = min(4096, rows)
    for r0 in sorted({0, rows - band}):
        want_out, want_sf = oracle.cast(x_host[r0:r0 + band], 'e4m3', (1, GROUP), round_sf=True, use_tma_aligned_col_major_sf=True,
                                        use_packed_ue8m0=True)
        got_out = out[r0:r0 + band].cpu().view(torch.uint8)
        got_sf = sf[r0:r0 + band].contiguous().cpu()
        ok = ok and torch.equal(got_out, want_out.view(torch.uint8)) and torch.equal(got_sf, want_sf.contiguous())
    return ok


def copy_ceiling_ms(torch, pipe, x_host, out_host, sf_host, device, steps: int, barrier) -> dict:
    """What the host <-> device links allow for the end-to-end call, measured two ways (all ranks at the same time):
    `pipeline`: the same chunked copies on the same streams as HostCastPipeline, without the kernels;
    `bulk`: one large host-to-device copy of the input and one device-to-host copy of the output, concurrently."""
    rows = x_host.shape[0]
    x_dev = torch.empty_like(x_host, device=device)
    out_dev = torch.empty(out_host.shape, dtype=torch.uint8, device=device)
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def bulk():
        cur = torch.cuda.current_stream(device)
        up.wait_stream(cur)
        down.wait_stream(cur)
        with torch.cuda.stream(up):
            x_dev.copy_(x_host, non_blocking=True)
        with torch.cuda.stream(down):
            out_host.view(torch.uint8).copy_(out_dev, non_blocking=True)
        cur.wait_stream(up)
        cur.wait_stream(down)

    def pipeline():
        cur = torch.cuda.current_stream(device)
        pipe.h2d.wait_stream(cur)
        pipe.d2h.wait_stream(cur)
        for i, r0 in enumerate(range(0, rows, pipe.chunk_rows)):
            n = min(pipe.chunk_rows, rows - r0)
            slot = i % pipe.depth
            with torch.cuda.stream(pipe.h2d):
                if i >= pipe.depth:
                    pipe.h2d.wait_event(pipe.ev_free[slot])
                pipe.x_dev[slot][:n].copy_(x_host[r0:r0 + n], non_blocking=True)
                pipe.ev_loaded[slot].record(pipe.h2d)
            with torch.cuda.stream(pipe.d2h):
                pipe.d2h.wait_event(pipe.ev_loaded[slot])
                out_host[r0:r0 + n].view(torch.uint8).copy_(pipe.out_dev[slot][:n], non_blocking=True)
                pipe.ev_free[slot].record(pipe.d2h)
        cur.wait_stream(pipe.d2h)

    ms_bulk, _, _, _ = time_steps(torch, bulk, steps, 2, barrier)
    ms_pipe, _, _, _ = time_steps(torch, pipeline, steps, 2, barrier)
    return {'bulk': ms_bulk / steps, 'pipeline': ms_pipe / steps}


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

    out_bytes_per_step = rows * HIDDEN + rows * (HIDDEN // GROUP)
    with ClockSampler(torch, local_rank) as sampler:
        ms, t0, t1, launch_mode = time_steps(torch, step, args.steps, args.warmup, barrier, graph_bytes_per_step=out_bytes_per_step)
    clocks = sampler.summary(t0, t1)
    if clocks['samples'] == 0:  # a timed region shorter than the sampling period: use the samples around it
        clocks = sampler.summary()

    # what the ranks wrote, checked against the CPU checker on the first and last band of every shard
    import oracle
    out_dev, sf_dev = step()
    parity_ok = shard_parity(torch, oracle, x_host, out_dev, sf_dev, rows)
    del out_dev, sf_dev

    # end to end through the host-buffer API
    out_host = torch.empty((rows, HIDDEN), dtype=torch.float8_e4m3fn, pin_memory=True)
    sf_host = torch.empty((HIDDEN // GROUP // 4, rows), dtype=torch.int32, pin_memory=True)
    chunk_rows = max(1024, min(4096, rows // 16 // 256 * 256))  # at least 16 chunks per call keep the ring busy
    pipe = host.HostCastPipeline(device, hidden=HIDDEN, max_rows=rows, chunk_rows=chunk_rows, depth=4)

    def e2e_step():
        pipe.per_token_cast_host(x_host, 'e4m3', GROUP, out_host, sf_host)

    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e, _, _, _ = time_steps(torch, e2e_step, e2e_steps, 3, barrier)
    e2e_parity = torch.equal(out_host[:chunk_rows].view(torch.uint8), step()[0][:chunk_rows].cpu().view(torch.uint8))
    ceiling = copy_ceiling_ms(torch, pipe, x_host, out_host, sf_host, device, max(1, min(args.steps, 3)), barrier)

    mine = torch.tensor([ms, ms_e2e, ceiling['bulk'], ceiling['pipeline'], 1.0 if (parity_ok and e2e_parity) else 0.0],
                        dtype=torch.float64, device=device)
    if world > 1:
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        table = torch.stack(everyone).cpu()
    else:
        table = mine.cpu().unsqueeze(0)
    ms, ms_e2e, ms_bulk, ms_pipe = (float(table[:, i].max()) for i in range(4))
    parity_all = bool(table[:, 4].min() > 0.5)
    per_rank = sorted(float(v) / args.steps for v in table[:, 0])

    if rank == 0:
        peak, peak_kind = hbm_peak()
        ms_per_step = ms / args.steps
        value = total_rows / (ms_per_step * 1e-3) / 1e6
        kernel_gbs = rows * bytes_per_token() / (ms_per_step * 1e-3) / 1e9  # per GPU: one launch per step on each rank
        e2e_value = total_rows / (ms_e2e / e2e_steps * 1e-3) / 1e6
        ceiling_value = total_rows / (max(min(ms_bulk, ms_pipe), 1e-9) * 1e-3) / 1e6  # the better of the two copy-only forms
        traffic = profiled_traffic()
        line = {
            'metric': 'per_token_cast_fp8_e4m3_g128_ue8m0_throughput', 'value': round(value, 2), 'unit': 'Mtokens/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms_per_step, 4),
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'config': workload_config(total_rows, world),
            'hbm_gbs': round(kernel_gbs * world, 1),
            'pct_of_8tbs': round(kernel_gbs / 8000.0 * 100, 1),
            'clocks': clocks,
            # device time per step of every rank: the spread between ranks and the per-launch cost, separately
            'ms_per_rank': {'min': round(per_rank[0], 4), 'median': round(statistics.median(per_rank), 4), 'max': round(per_rank[-1], 4)},
            'shard_parity': 'ok' if parity_all else 'MISMATCH',
            # bytes of all ranks together, like `value`
            'e2e': {'value': round(e2e_value, 3), 'unit': 'Mtokens/s', 'h2d_bytes_per_step': total_rows * HIDDEN * 2,
                    'd2h_bytes_per_step': total_rows * HIDDEN + total_rows * (HIDDEN // GROUP), 'steps': e2e_steps,
                    'api': 'tilekernels_b200.host.HostCastPipeline.per_token_cast_host (pinned host buffers)',
                    'chunk_rows': chunk_rows, 'depth': pipe.depth,
                    # the same bytes over the same links without any kernel, all ranks at once
                    'copy_ceiling': {'value': round(ceiling_value, 3), 'unit': 'Mtokens/s',
                                     'how': 'the same bytes over the same links without any kernel, all ranks at once; the better of two forms',
                                     'bulk_copies': round(total_rows / (max(ms_bulk, 1e-9) * 1e-3) / 1e6, 3),
                                     'pipeline_copies_only': round(total_rows / (max(ms_pipe, 1e-9) * 1e-3) / 1e6, 3)},
                    'frac_of_ceiling': round(e2e_value / ceiling_value, 3)},
            'gpu_launches': args.steps,
            'launch': launch_mode,
            'roofline': {'bound': 'hbm', 'achieved': round(kernel_gbs, 1), 'peak': peak, 'unit': 'GB/s',
                         'frac': round(kernel_gbs / peak, 4), 'peak_source': f'of {peak_kind}',
                         'traffic': None if traffic is None else traffic['dram_bytes_per_token'] * rows,
                         'traffic_source': None if traffic is None else
                         f"profiler capture at commit {traffic['captured_at_commit']} ({traffic['captured_rows']} rows), scaled by rows; not measured in this run",
                         'algorithmic_bytes_per_launch': rows * bytes_per_token(), 'kernel': 'group_cast_kernel<bf16,e4m3,LPG=8>'},
        }
        if world == 1:
            cores = os.cpu_count() or 1
            sample_rows = 32768
            line['cpu_baseline'] = {'value': round(oracle_rate(sample_rows, cores, repeats=3), 3), 'unit': 'Mtokens/s', 'cores': cores,
                                    'kind': 'port', 'sample': f'{sample_rows} of {TOTAL_ROWS} rows, best of 3', 'cpu': cpu_model()}
            if not args.no_ops:
                del x, pipe
                torch.cuda.empty_cache()
                line['ops'] = bench_other_ops(torch, quant, device, count_bytes)
                if args.records:
                    # one record per op in the form of the reference's benchmark plugin (kernel, operation, params,
                    # time_us, bandwidth_gbs, extras), one JSON object per line
                    with open(args.records, 'w') as f:
                        for r in line['ops']:
                            rec = {'kernel': r['kernel'], 'operation': r['operation'], 'params': dict(sorted(r['params'].items())),
                                   'time_us': r['time_us'], 'bandwidth_gbs': r['bandwidth_gbs'],
                                   'extras': {'copy_us': r['copy_us'], 'host_us_per_call': r['host_us_per_call']}}
                            f.write(json.dumps(rec) + '\n')
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
    ap.add_argument('--records', default='', help='also write the per-op table as JSONL records to this file')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
