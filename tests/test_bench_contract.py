"""The benchmark's reference arm runs without a GPU: its one JSON line must carry the keys the benchmark contract
names (the GPU arm prints the same line plus `roofline`, `clocks`, `ops`)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--rows', '1024', '--steps', '1',
                           '--warmup', '1'], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [line for line in proc.stdout.splitlines() if line.startswith('{')]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record['impl'] == 'reference' and record['n_gpus'] == 1 and record['steps'] == 1
    for key in ('metric', 'value', 'unit', 'warmup', 'ms_per_step', 'higher_is_better', 'scaling', 'vs_baseline', 'dtype', 'data',
                'config', 'cpu_baseline', 'e2e', 'gpu_launches'):
        assert key in record, key
    assert record['value'] > 0 and record['vs_baseline'] is None and record['gpu_launches'] == 0
    assert 'workload' in record['config']
    baseline = record['cpu_baseline']
    assert baseline['kind'] == 'port' and baseline['cores'] >= 1 and baseline['value'] == record['value'] and baseline['cpu']
    assert record['e2e'] == {'value': record['value'], 'unit': record['unit'], 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}
