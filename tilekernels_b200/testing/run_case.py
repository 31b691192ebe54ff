"""Run one benchmark workload a few times on cuda:0 -- the small, self-ending program that profiler captures
(ncu) are taken on.

    python -m tilekernels_b200.testing.run_case --op cfg5 --rows 32768 --launches 3

ops: cfg1 (per-token e4m3, fp32 scales), cfg2_block, cfg2_channel, cfg3 (SwiGLU + cast; cfg3_ue8m0 with power-of-two scales), cfg4_fp4, cfg4_e5m6,
cfg5 (per-token e4m3, ue8m0 scales), back_e4m3 / back_e5m6 (dequantisation of cfg4's tensor to bf16), bwd (SwiGLU
backward + cast on cfg3's tensor quantised with power-of-two scales), expand (row expansion of cfg1's FP8 cast with
ue8m0 scales to 8 positions per token), requant (per-token e4m3 cast of cfg4's tensor already quantised per 128x128 block
with ue8m0 scales), large_block / large_channel (the tile casts on cfg4's [32768, 7168] tensor), lossless (cfg4's tensor
as FP4 with 1x32 ue8m0 scales re-blocked to FP8 128x128), swiglu_channel (SwiGLU + per-channel cast + transpose on cfg3's
tensor), channel_fp8 (fused per-channel cast of cfg4's tensor as FP8 with fp32 group-128 scales).  --rows limits the row count (same per-row distribution).
"""
import argparse

import torch

from tilekernels_b200 import moe, quant
from tilekernels_b200.testing import count_bytes, make_config_input

OPS = {
    'cfg1': ('cfg1', lambda x: quant.per_token_cast(x, 'e4m3', 128)),
    'cfg2_block': ('cfg2', lambda x: quant.per_block_cast(x, 'e4m3', (128, 128))),
    'cfg2_channel': ('cfg2', lambda x: quant.per_channel_cast(x, 'e4m3', 128)),
    'cfg3': ('cfg3', lambda x: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128)),
    'cfg3_ue8m0': ('cfg3', lambda x: quant.swiglu_forward_and_per_token_cast(x, 'e4m3', 128, use_tma_aligned_col_major_sf=True, round_sf=True,
                                                                              use_packed_ue8m0=True)),
    'cfg4_fp4': ('cfg4', lambda x: quant.per_token_cast(x, 'e2m1', 32, None, True, True, True)),
    'cfg4_e5m6': ('cfg4', lambda x: quant.per_token_cast(x, 'e5m6', x.shape[1])),
    'back_e4m3': ('cfg4', lambda q: (quant.cast_back(q, 'bf16', (1, 128)),)),
    'back_e5m6': ('cfg4', lambda q: (quant.cast_back_e5m6(q, 'bf16', (1, q[0].shape[1] // 3 * 2)),)),
    'bwd': ('cfg3', lambda a: quant.swiglu_backward_and_per_token_cast(*a, 128, True)),
    'expand': ('cfg1', lambda a: moe.expand_to_fused_with_sf(a[0], 128, a[1], a[2], True)),
    'cfg5': ('cfg5', lambda x: quant.per_token_cast(x, 'e4m3', 128, None, True, True, True)),
    'requant': ('cfg4', lambda q: quant.per_token_cast(q, 'e4m3', 128, (128, 128), True, True, True)),
    'large_block': ('cfg4', lambda x: quant.per_block_cast(x, 'e4m3', (128, 128))),
    'large_channel': ('cfg4', lambda x: quant.per_channel_cast(x, 'e4m3', 128)),
    'lossless': ('cfg4', lambda q: quant.per_block_cast_lossless(q, 'e4m3', (1, 32), (128, 128), True, True, True)),
    'channel_fp8': ('cfg4', lambda q: quant.per_channel_cast_fused(q, 'e4m3', 128, False, 128)),
    'swiglu_channel': ('cfg3', lambda x: quant.swiglu_forward_and_per_channel_cast_and_transpose(x, 'e4m3', 128)),
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
    elif args.op == 'channel_fp8':
        x = quant.per_token_cast(x, 'e4m3', 128)
    elif args.op == 'lossless':
        x = quant.per_token_cast(x, 'e2m1', 32, None, True, True, True)
    elif args.op == 'requant':
        x = quant.per_block_cast(x, 'e4m3', (128, 128), True, True, True)
    elif args.op == 'back_e5m6':
        x = quant.per_token_cast(x, 'e5m6', x.shape[1])
    elif args.op == 'bwd':
        rows, hidden = x.shape[0], x.shape[1] // 2
        g = torch.Generator().manual_seed(11)
        pos = torch.randperm(rows, generator=g).to(torch.int32)
        token_topk_to_pos = torch.empty(rows, dtype=torch.int32)
        token_topk_to_pos[pos.long()] = torch.arange(rows, dtype=torch.int32)
        x = (quant.per_token_cast(x, 'e4m3', 128, round_sf=True), torch.randn((rows, hidden), generator=g).to(torch.bfloat16).cuda(),
             torch.rand((rows // 8, 8), generator=g).cuda(), pos.cuda(), token_topk_to_pos.view(-1, 8).cuda())
    elif args.op == 'expand':
        q, sf = quant.per_token_cast(x, 'e4m3', 128, None, True, True, True)
        positions = torch.randperm(x.shape[0] * 8, generator=torch.Generator().manual_seed(13)).to(torch.int32)
        x = ((q, sf.contiguous()), positions.view(-1, 8).cuda(), torch.zeros(x.shape[0] * 8, dtype=torch.int32, device='cuda'))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(args.launches):
        if i == args.launches - 1:
            start.record()
        out = op(x)
    stop.record()
    torch.cuda.synchronize()
    nbytes = count_bytes(x, out)
    rows = (x[0][0] if isinstance(x[0], tuple) else x[0]).shape[0] if isinstance(x, tuple) else x.shape[0]
    us = start.elapsed_time(stop) * 1e3
    print(f'{args.op}: rows={rows} bytes={nbytes} last launch {us:.1f} us -> {nbytes / us / 1e3:.0f} GB/s (includes host launch overhead)')


if __name__ == '__main__':
    main()
