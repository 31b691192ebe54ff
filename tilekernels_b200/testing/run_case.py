"""Run one benchmark workload a few times on cuda:0 -- the small, self-ending program that profiler captures
(ncu) are taken on.

    python -m tilekernels_b200.testing.run_case --op cfg5 --rows 32768 --launches 3

ops: cfg1 (per-token e4m3, fp32 scales), cfg2_block, cfg2_channel, cfg3 (SwiGLU + cast), cfg4_fp4, cfg4_e5m6,
cfg5 (per-token e4m3, ue8m0 scales), back_e4m3 / back_e5m6 (dequantisation of cfg4's tensor to bf16).  --rows limits
the row count (same per-row distribution).
"""
import argparse

import torch

from tilekernels_b200 import quant
from tilekernels_b200.testing import make_config_input

OPS = {
    'cfg1': ('cfg1', lambda x: quant.per_token_cast(x, 'e4m3', 128)),
    'cfg2_block': ('cfg2', lambda x: quant.per_block_cast(x, 'e4m3', (128, 128))),
    'cfg2_channel': ('cfg2', lambda x: quant.per_channel_cast(x, 'e4m3', 128)),
    'cfg3': ('cfg3', lambda x: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128)),
    'cfg4_fp4': ('cfg4', lambda x: quant.per_token_cast(x, 'e2m1', 32, None, True, True, True)),
    'cfg4_e5m6': ('cfg4', lambda x: quant.per_token_cast(x, 'e5m6', x.shape[1])),
    'back_e4m3': ('cfg4', lambda q: (quant.cast_back(q, 'bf16', (1, 128)),)),
    'back_e5m6': ('cfg4', lambda q: (quant.cast_back_e5m6(q, 'bf16', (1, q[0].shape[1] // 3 * 2)),)),
    'cfg5': ('cfg5', lambda x: quant.per_token_cast(x, 'e4m3', 128, None, True, True, True)),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--op', required=True, choices=sorted(OPS))
    ap.add_argument('--rows', type=int, default=None)
    ap.add_argument('--launches', type=int, default=3)
    args = ap.parse_args()
    cfg, op = OPS[args.op]
    x = make_config_input(cfg, args.rows).cuda()
    if args.op == 'back_e4m3':
        x = quant.per_token_cast(x, 'e4m3', 128)
    elif args.op == 'back_e5m6':
        x = quant.per_token_cast(x, 'e5m6', x.shape[1])
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(args.launches):
        if i == args.launches - 1:
            start.record()
        out = op(x)
    stop.record()
    torch.cuda.synchronize()
    tensors = (list(x) if isinstance(x, tuple) else [x]) + list(out)
    nbytes = sum(t.numel() * t.element_size() for t in tensors)
    rows = tensors[0].shape[0]
    us = start.elapsed_time(stop) * 1e3
    print(f'{args.op}: rows={rows} bytes={nbytes} last launch {us:.1f} us -> {nbytes / us / 1e3:.0f} GB/s (includes host launch overhead)')


if __name__ == '__main__':
    main()
