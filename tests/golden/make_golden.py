"""Generate the golden fixtures of this folder from the reference implementation.

Run in a container that has the reference checkout (it is imported, never copied):

    PYTHONPATH=/path/to/TileKernels python tests/golden/make_golden.py

It calls the reference's own PyTorch implementation (tile_kernels.torch.cast,
cast_to_e5m6, swiglu_forward, cast_back) on seeded CPU inputs and stores inputs and
outputs as raw bytes in small .npz files, plus SHA-256 digests of the reference
outputs for reduced-row versions of the five benchmark workloads
(config_digests.json).  The tests compare the CPU oracle and the CUDA kernels
with these files; nothing at test time needs the reference.
"""
import hashlib
import json
import os
import sys

os.environ.setdefault('TORCHDYNAMO_DISABLE', '1')  # see gen_swiglu_backward

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tile_kernels.torch import cast, cast_back, cast_to_e5m6, swiglu_forward  # noqa: E402  (the reference)
from tile_kernels.torch.cast import convert_to_e2m1_bits  # noqa: E402
from tile_kernels.torch.cast_e5m6 import _cast_to_e5m6  # noqa: E402

from tilekernels_b200.testing.generator import make_config_input  # noqa: E402

FLAG_SETS = [(False, False, False), (False, True, False), (True, True, True)]  # (col_major, round_sf, ue8m0)


def raw(t: torch.Tensor) -> np.ndarray:
    dense = torch.empty(t.shape, dtype=t.dtype)
    dense.copy_(t)
    return dense.flatten().view(torch.uint8).numpy().copy()


def meta(t: torch.Tensor) -> str:
    return json.dumps({'dtype': str(t.dtype).replace('torch.', ''), 'shape': list(t.shape), 'stride': list(t.stride())})


def put(store: dict, key: str, t: torch.Tensor) -> None:
    store[key + '.bytes'] = raw(t)
    store[key + '.meta'] = np.array(meta(t))


def special_rows(x: torch.Tensor) -> torch.Tensor:
    """Overwrite the first rows with corner cases: zeros, signed zeros, huge, tiny, outliers."""
    x = x.clone()
    big = 3.3895e38 if x.dtype == torch.bfloat16 else 3.0e38
    x[0] = 0
    x[1] = -0.0
    x[2, ::2] = big
    x[2, 1::2] = -big
    x[3] = 1e-30
    x[4] = x[4] * 1e-3
    x[5, 7] = 1000.0
    x[6] = 6.0
    x[7] = torch.linspace(-8, 8, x.shape[1]).to(x.dtype)
    return x


def gen_cast() -> None:
    store = {}
    g = torch.Generator().manual_seed(1234)
    inputs = {
        'bf16_33x320': special_rows(torch.randn((33, 320), generator=g)).to(torch.bfloat16),
        'fp32_9x192': special_rows(torch.randn((9, 192), generator=g)),
        'bf16_130x128': torch.randn((130, 128), generator=g).to(torch.bfloat16),
    }
    for name, x in inputs.items():
        put(store, f'{name}/x', x)
        T, H = x.shape
        for fmt in ('e4m3', 'e2m1'):
            for bs in ((1, 32), (1, 64), (1, 128), (1, H), (128, 128), (32, 32), (128, 1)):
                if bs == (128, 1) and fmt == 'e2m1':
                    continue
                for col, rnd, ue in FLAG_SETS:
                    if bs == (128, 1) and col:
                        continue
                    out, sf = cast(x, fmt, bs, round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
                    key = f'{name}/{fmt}/{bs[0]}x{bs[1]}/{int(col)}{int(rnd)}{int(ue)}'
                    put(store, key + '/out', out)
                    put(store, key + '/sf', sf)
                    if not col:
                        put(store, key + '/out_pre', cast(x, fmt, bs, sf=sf))
                        if rnd and name == 'bf16_33x320':
                            put(store, key + '/back', cast_back((out, sf), 'fp32', bs))
    np.savez_compressed(os.path.join(HERE, 'cast.npz'), **store)


def gen_e5m6() -> None:
    store = {}
    g = torch.Generator().manual_seed(4321)
    inputs = {
        'bf16_33x320': special_rows(torch.randn((33, 320), generator=g)).to(torch.bfloat16),
        'fp32_9x192': special_rows(torch.randn((9, 192), generator=g)),
    }
    for value, tag in ((2.0 ** -20, 'minsub'), (2.0 ** -14 * 63 / 64, 'maxsub'), (2.0 ** -14, 'minnorm')):
        x = torch.full((5, 64), value, dtype=torch.bfloat16)
        x[:, -1] = 65024.0
        inputs[f'bf16_special_{tag}'] = x
        inputs[f'fp32_special_{tag}'] = x.float().fill_(value).index_fill_(1, torch.tensor([63]), 65024.0)
    for name, x in inputs.items():
        put(store, f'{name}/x', x)
        for col, rnd, ue in FLAG_SETS:
            out, sf = cast_to_e5m6(x, x.shape[1], col, rnd, ue)
            key = f'{name}/{int(col)}{int(rnd)}{int(ue)}'
            put(store, key + '/out', out)
            put(store, key + '/sf', sf)
    # element-level known answers: codes of a sweep of floats, before packing
    v = torch.cat([torch.randn(4096, generator=g) * s for s in (1e-6, 1e-4, 1e-2, 1.0, 100.0, 20000.0)]).clamp(-65024, 65024)
    v = torch.cat([v, torch.tensor([0.0, -0.0, 65024.0, -65024.0, 2.0 ** -20, 2.0 ** -21, 2.0 ** -14, 1.0 + 2.0 ** -7, 1.0 + 3 * 2.0 ** -7])])
    v = torch.cat([v, torch.zeros(8 - v.numel() % 8 if v.numel() % 8 else 0)])
    put(store, 'kat/x', v)
    put(store, 'kat/words', _cast_to_e5m6(v.view(1, -1)))
    np.savez_compressed(os.path.join(HERE, 'e5m6.npz'), **store)


def gen_e2m1_kat() -> None:
    store = {}
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    vals = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 7.0, 1e9, 1e-9]
    pts = []
    for m in mids + vals:
        t = torch.tensor([m], dtype=torch.float32)
        pts += [t, torch.nextafter(t, torch.tensor([10.0])), torch.nextafter(t, torch.tensor([-10.0]))]
    g = torch.Generator().manual_seed(99)
    v = torch.cat(pts + [torch.randn(8192, generator=g) * 2.5])
    v = torch.cat([v, -v])
    put(store, 'x', v)
    put(store, 'codes', convert_to_e2m1_bits(v, 6.0, 'cpu'))
    np.savez_compressed(os.path.join(HERE, 'e2m1_kat.npz'), **store)


def gen_swiglu() -> None:
    """Reference outputs of cast(swiglu_forward(x), ...).  torch's CPU exp differs from this project's
    exp in the last bit of a few percent of the activations, so these are compared with a tolerance."""
    store = {}
    g = torch.Generator().manual_seed(777)
    T, H = 48, 256
    x = torch.randn((T, 2 * H), generator=g).to(torch.bfloat16)
    put(store, 'x', x)
    pos = torch.randperm(T, generator=g).to(torch.int32)
    pos[::7] = -1
    w = torch.rand((8, 6), generator=g)
    put(store, 'pos_to_token_topk', pos)
    put(store, 'topk_weights', w)
    for with_w in (False, True):
        for clamp in (None, 0.5):
            counts = torch.zeros(3, dtype=torch.int64)
            y = swiglu_forward(x, pos if with_w else None, w if with_w else None, clamp, counts if clamp else None)
            key0 = f'w{int(with_w)}/c{clamp}'
            put(store, key0 + '/y', y)
            put(store, key0 + '/counts', counts)
            for G in (128, H):
                for col, rnd, ue in FLAG_SETS:
                    if G == H and col:
                        continue
                    out, sf = cast(y, 'e4m3', (1, G), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
                    key = f'{key0}/g{G}/{int(col)}{int(rnd)}{int(ue)}'
                    put(store, key + '/out', out)
                    put(store, key + '/sf', sf)
    np.savez_compressed(os.path.join(HERE, 'swiglu.npz'), **store)


def gen_swiglu_cfg3() -> None:
    """The fused SwiGLU cast on the benchmark workload itself (cfg3, [16384, 4096] bf16 ~ N(0,1), gate | up halves
    of 2048) at reduced row counts: cast(swiglu_forward(x), 'e4m3', (1, 128)) from the reference (the sequence of
    tests/quant/test_swiglu_forward_and_per_token_cast.py:91-110, formula tile_kernels/torch/swiglu.py:61-75).
    Large enough for the tolerance on the codes (at most one code apart on at most 1e-4 of the elements) to mean
    something: 1024 rows = 2.1 M activations = 16384 scale groups for the default flags; 512 rows for the
    power-of-two scales in the packed-ue8m0 layout; 256 rows for the variant with row weights, clamp and clamp
    counters.  The
    inputs are not stored: make_config_input('cfg3', rows) regenerates them and their digest is checked."""
    store = {}
    x = make_config_input('cfg3', 1024)
    store['x1024.sha256'] = np.array(sha(x))
    out, sf = cast(swiglu_forward(x), 'e4m3', (1, 128))
    put(store, 'plain/000/out', out)
    put(store, 'plain/000/sf', sf)
    x = x[:512]
    y = swiglu_forward(x)
    out, sf = cast(y, 'e4m3', (1, 128), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    put(store, 'plain/111/out', out)
    put(store, 'plain/111/sf', sf)
    # row weights (a permutation of (token, k) pairs with holes), clamp 2.5 (about 0.6 % of the gates, 1.2 % of the
    # up values) and the three clamp counters
    x = x[:256]
    g = torch.Generator().manual_seed(31)
    pos = torch.randperm(256, generator=g).to(torch.int32)
    pos[::13] = -1
    w = torch.rand((32, 8), generator=g)
    put(store, 'moe/pos_to_token_topk', pos)
    put(store, 'moe/topk_weights', w)
    counts = torch.zeros(3, dtype=torch.int64)
    y = swiglu_forward(x, pos, w, 2.5, counts)
    put(store, 'moe/counts', counts)
    for col, rnd, ue in ((False, False, False), (True, True, True)):
        out, sf = cast(y, 'e4m3', (1, 128), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
        key = f'moe/{int(col)}{int(rnd)}{int(ue)}'
        put(store, key + '/out', out)
        put(store, key + '/sf', sf)
    np.savez_compressed(os.path.join(HERE, 'swiglu_cfg3.npz'), **store)


def gen_requant() -> None:
    """Already quantized inputs (FP8 / FP4 data + scales in every layout) cast again per token, and the fused
    per-channel cast with FP8 input and row gather (reference: tile_kernels/torch/cast.py:86-97,
    tile_kernels/torch/per_channel_cast_fused.py:9-44)."""
    from tile_kernels.torch.per_channel_cast_fused import per_channel_cast_fused
    store = {}
    g = torch.Generator().manual_seed(2468)
    x = torch.randn((40, 256), generator=g).to(torch.bfloat16)
    x[3] = 0
    x[5] *= 300
    put(store, 'x', x)
    for in_fmt in ('e4m3', 'e2m1'):
        for xbs in ((128, 128), (32, 32)):
            for col, rnd, ue in ((False, True, False), (True, True, True)):
                q, qsf = cast(x, in_fmt, xbs, round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
                key_in = f'{in_fmt}/{xbs[0]}/{int(col)}{int(rnd)}{int(ue)}'
                put(store, key_in + '/q', q)
                put(store, key_in + '/qsf', qsf)
                for fmt in ('e4m3', 'e2m1'):
                    for G in (32, 128):
                        out, sf = cast((q, qsf), fmt, (1, G), x_block_size=xbs, round_sf=rnd, use_tma_aligned_col_major_sf=col,
                                       use_packed_ue8m0=ue)
                        put(store, f'{key_in}/{fmt}/g{G}/out', out)
                        put(store, f'{key_in}/{fmt}/g{G}/sf', sf)
    # fused per-channel cast: plain and FP8 + per-token-group scales, with and without gather
    T, H = 128, 256
    xb = torch.randn((T, H), generator=g).to(torch.bfloat16)
    q8, s8 = cast(xb, 'e4m3', (1, 128), round_sf=False)
    pos = torch.randint(0, T, (144,), generator=g, dtype=torch.int32)
    pos[::9] = -1
    put(store, 'pc/x', xb)
    put(store, 'pc/q8', q8)
    put(store, 'pc/s8', s8)
    put(store, 'pc/pos', pos)
    for rnd in (False, True):
        for src in ('bf16', 'fp8'):
            for gather in (False, True):
                xin = xb if src == 'bf16' else (q8, s8)
                out, sf = per_channel_cast_fused(xin, 128, None if src == 'bf16' else 128, rnd, pos if gather else None)
                put(store, f'pc/{src}/r{int(rnd)}/g{int(gather)}/out', out)
                put(store, f'pc/{src}/r{int(rnd)}/g{int(gather)}/sf', sf)
    np.savez_compressed(os.path.join(HERE, 'requant.npz'), **store)


def gen_cast_back() -> None:
    """Dequantisation (reference: tile_kernels/torch/cast.py:40-59, cast_e5m6.py:221-258).  Only the fp32 result is
    stored; the bf16 result is by definition that tensor rounded to bfloat16."""
    from tile_kernels.torch import cast_back_from_e5m6
    store = {}
    g = torch.Generator().manual_seed(1357)
    x = torch.randn((40, 128), generator=g).to(torch.bfloat16)
    x[2] = 0
    x[7] *= 1000
    put(store, 'x', x)
    for fmt in ('e4m3', 'e2m1'):
        for bs in ((1, 32), (1, 128), (128, 128), (32, 32)):
            for col, rnd, ue in ((False, True, False), (True, True, True)):
                q, qsf = cast(x, fmt, bs, round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
                key = f'{fmt}/{bs[0]}x{bs[1]}/{int(col)}{int(rnd)}{int(ue)}'
                put(store, key + '/q', q)
                put(store, key + '/qsf', qsf)
                put(store, key + '/back', cast_back((q, qsf), 'fp32', bs))
    for col, rnd, ue in FLAG_SETS:
        q, qsf = cast_to_e5m6(x, 128, col, rnd, ue)
        key = f'e5m6/{int(col)}{int(rnd)}{int(ue)}'
        put(store, key + '/q', q)
        put(store, key + '/qsf', qsf)
        put(store, key + '/back', cast_back_from_e5m6((q, qsf), 'fp32', (1, 128)))
    np.savez_compressed(os.path.join(HERE, 'cast_back.npz'), **store)


def gen_swiglu_backward() -> None:
    """Reference outputs of swiglu_backward followed by cast (reference: tile_kernels/torch/swiglu.py:98-226, the
    sequence of tests/quant/test_swiglu_backward_and_per_token_cast.py:83-102).

    The reference routes 1 + x * (1 - s) through a torch.compile'd helper so that it becomes ONE fused
    multiply-add (swiglu.py:91-95).  torch.compile has no working C++ back end in the container this runs in,
    so the script is run with TORCHDYNAMO_DISABLE=1 and that helper is replaced by an exact emulation of the
    fused operation: the product of two floats is exact in double, the sum is rounded once to double and once
    to float."""
    import tile_kernels.torch.swiglu as ref_swiglu

    def fma(a, b, c):
        return (a.double() * (b.double() if torch.is_tensor(b) else b) + c).float()

    ref_swiglu.elementwise_fma = fma
    store = {}
    g = torch.Generator().manual_seed(4242)
    T, H, num_tokens, topk = 24, 384, 8, 4
    x = (torch.randn((T, 2 * H), generator=g) * 2).to(torch.bfloat16)
    x[3] = 0
    x[4] *= 40                      # saturated gates: exp under- and overflows, s = 0 or 1
    d = torch.randn((T, H), generator=g).to(torch.bfloat16)
    w = torch.rand((num_tokens, topk), generator=g)
    perm = torch.randperm(num_tokens * topk, generator=g)[:T].to(torch.int32)
    perm[::9] = -1                  # unused expanded positions
    t2p = torch.full((num_tokens * topk,), -1, dtype=torch.int32)
    for row, index in enumerate(perm.tolist()):
        if index >= 0:
            t2p[index] = row
    t2p = t2p.view(num_tokens, topk)
    put(store, 'grad_out', d)
    put(store, 'weight', w)
    put(store, 'pos_to_token_topk', perm)
    put(store, 'token_topk_to_pos', t2p)
    for G in (32, 128):
        q, qsf = cast(x, 'e4m3', (1, G))
        put(store, f'g{G}/q', q)
        put(store, f'g{G}/qsf', qsf)
        for clamp in (None, 10.0, 0.5):
            out, x_grad, w_grad = ref_swiglu.swiglu_backward((q, qsf), d, w, perm, t2p, G, clamp)
            key = f'g{G}/c{clamp}'
            put(store, key + '/out', out.to(torch.bfloat16))
            put(store, key + '/x_grad', x_grad.to(torch.bfloat16))
            put(store, key + '/weight_grad', w_grad)
            for rnd in (False, True):
                o8, s8 = cast(x_grad, 'e4m3', (1, G), round_sf=rnd)
                put(store, f'{key}/r{int(rnd)}/fp8', o8)
                put(store, f'{key}/r{int(rnd)}/sf', s8)
    np.savez_compressed(os.path.join(HERE, 'swiglu_backward.npz'), **store)


def gen_expand() -> None:
    """Row expansion into the fused expert layout (reference: tile_kernels/torch/expand_to_fused.py:6-91), plain and
    with scale factors in the three layouts the reference's test uses."""
    from tile_kernels.torch.expand_to_fused import expand_to_fused, expand_to_fused_with_sf
    store = {}
    g = torch.Generator().manual_seed(8642)
    num_tokens, topk, hidden, num_expanded = 19, 3, 256, 70
    x = torch.randn((num_tokens, hidden), generator=g).to(torch.bfloat16)
    routed = torch.rand(num_tokens * topk, generator=g) > 0.25
    positions = torch.randperm(num_expanded, generator=g)[:int(routed.sum())].to(torch.int32)
    t2p = torch.full((num_tokens * topk,), -1, dtype=torch.int32)
    t2p[routed] = positions
    t2p = t2p.view(num_tokens, topk)
    p2e = torch.full((num_expanded,), -1, dtype=torch.int32)
    p2e[positions.long()] = torch.randint(0, 8, (positions.numel(),), generator=g, dtype=torch.int32)
    put(store, 'x', x)
    put(store, 'token_topk_to_pos', t2p)
    put(store, 'pos_to_expert', p2e)
    put(store, 'plain', expand_to_fused(x, t2p, p2e))
    for G in (32, 128):
        for col, rnd, ue in ((False, True, False), (True, True, False), (True, True, True)):
            q, qsf = cast(x, 'e4m3', (1, G), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
            qsf = qsf.contiguous()
            out, out_sf = expand_to_fused_with_sf((q, qsf), G, t2p, p2e, col)
            key = f'g{G}/{int(col)}{int(rnd)}{int(ue)}'
            put(store, key + '/q', q)
            put(store, key + '/qsf', qsf)
            put(store, key + '/out', out)
            put(store, key + '/out_sf', out_sf)
    np.savez_compressed(os.path.join(HERE, 'expand.npz'), **store)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(raw(t).tobytes()).hexdigest()


def gen_config_digests() -> None:
    """Reference outputs of the five benchmark workloads at reduced row counts, as digests."""
    d = {}

    def add(name, x, out, sf):
        d[name] = {'rows': x.shape[0], 'x': sha(x), 'out': sha(out), 'sf': sha(sf), 'sf_meta': json.loads(meta(sf))}

    x = make_config_input('cfg1', 1280)
    add('cfg1_per_token_e4m3_g128', x, *cast(x, 'e4m3', (1, 128)))
    add('cfg1_per_token_e4m3_g128_round', x, *cast(x, 'e4m3', (1, 128), round_sf=True))
    x = make_config_input('cfg2', 1024)
    add('cfg2_per_block_128x128', x, *cast(x, 'e4m3', (128, 128)))
    add('cfg2_per_channel_128', x, *cast(x, 'e4m3', (128, 1)))
    x = make_config_input('cfg4', 512)
    add('cfg4_fp4_g32_ue8m0', x, *cast(x, 'e2m1', (1, 32), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True))
    add('cfg4_e5m6', x, *cast_to_e5m6(x, x.shape[1]))
    x = make_config_input('cfg5', 1024)
    add('cfg5_per_token_e4m3_g128_ue8m0', x, *cast(x, 'e4m3', (1, 128), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True))
    with open(os.path.join(HERE, 'config_digests.json'), 'w') as f:
        json.dump(d, f, indent=1, sort_keys=True)


if __name__ == '__main__':
    torch.set_num_threads(8)
    generators = {'cast': gen_cast, 'e5m6': gen_e5m6, 'e2m1_kat': gen_e2m1_kat, 'swiglu': gen_swiglu, 'swiglu_cfg3': gen_swiglu_cfg3, 'requant': gen_requant,
                  'cast_back': gen_cast_back, 'swiglu_backward': gen_swiglu_backward, 'expand': gen_expand, 'config_digests': gen_config_digests}
    for name in (sys.argv[1:] or list(generators)):   # optional arguments: the fixtures to (re)generate
        generators[name]()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
