"""The CPU oracle against fixtures produced by the reference's own PyTorch implementation
(tests/golden/make_golden.py).  This is what pins the oracle; the GPU tests then compare
the CUDA kernels with the oracle."""
import hashlib
import json
import os

import pytest
import torch

from helpers import FLAG_SETS, GOLDEN, flags_id, golden, golden_tensor
from tilekernels_b200.testing import assert_equal, make_config_input

CAST_INPUTS = ['bf16_33x320', 'fp32_9x192', 'bf16_130x128']
BLOCKS = [(1, 32), (1, 64), (1, 128), (1, 0), (128, 128), (32, 32), (128, 1)]  # 0 = hidden


def _cast_cases():
    for name in CAST_INPUTS:
        for fmt in ('e4m3', 'e2m1'):
            for bs in BLOCKS:
                if bs == (128, 1) and fmt == 'e2m1':
                    continue
                for flags in FLAG_SETS:
                    if bs == (128, 1) and flags[0]:
                        continue
                    yield pytest.param(name, fmt, bs, flags, id=f'{name}-{fmt}-{bs[0]}x{bs[1]}-{flags_id(flags)}')


@pytest.mark.parametrize('name,fmt,bs,flags', list(_cast_cases()))
def test_cast_matches_reference(oracle, name, fmt, bs, flags):
    store = golden('cast')
    x = golden_tensor(store, f'{name}/x')
    bs = (bs[0], bs[1] or x.shape[1])
    col, rnd, ue = flags
    key = f'{name}/{fmt}/{bs[0]}x{bs[1]}/{flags_id(flags)}'
    out, sf = oracle.cast(x, fmt, bs, round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    assert_equal(out, golden_tensor(store, key + '/out'))
    assert_equal(sf, golden_tensor(store, key + '/sf'))
    if not col:
        assert_equal(oracle.cast(x, fmt, bs, sf=sf), golden_tensor(store, key + '/out_pre'))
        if key + '/back.meta' in store:
            assert_equal(oracle.cast_back((out, sf), 'fp32', bs), golden_tensor(store, key + '/back'))


def test_cast_empty_shapes(oracle):
    # shapes/strides of the zero-token case (reference: tile_kernels/torch/cast.py:109-123)
    x = torch.empty((0, 256), dtype=torch.bfloat16)
    out, sf = oracle.cast(x, 'e4m3', (1, 128))
    assert out.shape == (0, 256) and sf.shape == (0, 2) and sf.dtype == torch.float32
    out, sf = oracle.cast(x, 'e2m1', (1, 32), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    assert out.shape == (0, 128) and out.dtype == torch.int8 and sf.shape == (0, 2) and sf.dtype == torch.int32


E5M6_INPUTS = ['bf16_33x320', 'fp32_9x192'] + [f'{d}_special_{t}' for d in ('bf16', 'fp32') for t in ('minsub', 'maxsub', 'minnorm')]


@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('name', E5M6_INPUTS)
def test_e5m6_matches_reference(oracle, name, flags):
    store = golden('e5m6')
    x = golden_tensor(store, f'{name}/x')
    col, rnd, ue = flags
    out, sf = oracle.cast_to_e5m6(x, x.shape[1], col, rnd, ue)
    key = f'{name}/{flags_id(flags)}'
    assert_equal(out, golden_tensor(store, key + '/out'))
    assert_equal(sf, golden_tensor(store, key + '/sf'))


def test_e5m6_element_codes(oracle):
    store = golden('e5m6')
    v = golden_tensor(store, 'kat/x')
    words = golden_tensor(store, 'kat/words').view(torch.int32).view(-1, 3).to(torch.int64) & 0xFFFFFFFF
    c = oracle.convert_array(v, 'e5m6').view(-1, 8).to(torch.int64)
    w0 = (c[:, 0] << 20) | (c[:, 1] << 8) | (c[:, 2] >> 4)
    w1 = ((c[:, 2] << 28) | (c[:, 3] << 16) | (c[:, 4] << 4) | (c[:, 5] >> 8)) & 0xFFFFFFFF
    w2 = ((c[:, 5] << 24) | (c[:, 6] << 12) | c[:, 7]) & 0xFFFFFFFF
    assert torch.equal(torch.stack([w0, w1, w2], dim=1), words)


def test_e2m1_element_codes(oracle):
    # every rounding midpoint of e2m1 with its two float neighbours, both signs, plus random values
    store = golden('e2m1_kat')
    v = golden_tensor(store, 'x')
    assert torch.equal(oracle.convert_array(v, 'e2m1'), golden_tensor(store, 'codes'))


def _swiglu_cases():
    for with_w in (False, True):
        for clamp in (None, 0.5):
            for G in (128, 256):
                for flags in FLAG_SETS:
                    if G == 256 and flags[0]:
                        continue
                    yield pytest.param(with_w, clamp, G, flags, id=f'w{int(with_w)}-c{clamp}-g{G}-{flags_id(flags)}')


@pytest.mark.parametrize('with_w,clamp,G,flags', list(_swiglu_cases()))
def test_swiglu_cast_close_to_reference(oracle, with_w, clamp, G, flags):
    """The fused SwiGLU cast differs from the reference in one place, exp(): the reference uses torch's
    (CPU: a vector library; CUDA: expf), this project an FMA-only routine shared by the oracle and the
    kernel.  Each is within 1 ulp of exp, so a few percent of the fp32 activations differ in the last
    bit.  Tolerances: power-of-two scales identical; fp32 scales equal or 1 ulp apart; FP8 codes at
    most 1 code apart on at most 1e-4 of the elements (3e-3 when a 1-ulp scale difference moves a
    whole group's products); clamp counters identical."""
    store = golden('swiglu')
    x = golden_tensor(store, 'x')
    pos = golden_tensor(store, 'pos_to_token_topk') if with_w else None
    w = golden_tensor(store, 'topk_weights') if with_w else None
    counts = torch.zeros(3, dtype=torch.int64)
    y = oracle.swiglu_forward(x, pos, w, clamp, counts if clamp else None)
    key0 = f'w{int(with_w)}/c{clamp}'
    y_ref = golden_tensor(store, key0 + '/y')
    assert torch.equal(counts, golden_tensor(store, key0 + '/counts'))
    ulp = (y.view(torch.int32) - y_ref.view(torch.int32)).abs()
    assert ulp.max().item() <= 4 and (ulp > 0).float().mean().item() < 0.05  # 1 ulp in exp, carried through / and two *

    col, rnd, ue = flags
    out, sf = oracle.cast(y, 'e4m3', (1, G), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    key = f'{key0}/g{G}/{flags_id(flags)}'
    out_ref, sf_ref = golden_tensor(store, key + '/out'), golden_tensor(store, key + '/sf')
    assert sf.dtype == sf_ref.dtype and sf.shape == sf_ref.shape
    if rnd:
        assert_equal(sf, sf_ref)
        code_budget = 1e-4
    else:
        d = (sf.clone().view(torch.int32) - sf_ref.clone().view(torch.int32)).abs()
        assert d.max().item() <= 1
        code_budget = 1e-4 if d.max().item() == 0 else 3e-3
    a, b = out.view(torch.uint8).to(torch.int32), out_ref.view(torch.uint8).to(torch.int32)
    diff = (a - b).abs()
    assert diff.max().item() <= 1
    assert (diff > 0).float().mean().item() <= code_budget
    # dequantised values agree to the format's step (one e4m3 code = 2^-3 relative)
    dq = out.float() * oracle.sf_to_float(sf).repeat_interleave(G, dim=1)[:, :out.shape[1]]
    dq_ref = out_ref.float() * oracle.sf_to_float(sf_ref).repeat_interleave(G, dim=1)[:, :out.shape[1]]
    same = diff == 0
    rel = ((dq - dq_ref).abs() / dq_ref.abs().clamp_min(1e-30))[same]
    assert rel.numel() == 0 or rel.max().item() <= 1e-3


def _requant_cases():
    for in_fmt in ('e4m3', 'e2m1'):
        for xb in (128, 32):
            for flags in ((False, True, False), (True, True, True)):
                for fmt in ('e4m3', 'e2m1'):
                    for G in (32, 128):
                        yield pytest.param(in_fmt, xb, flags, fmt, G, id=f'{in_fmt}-b{xb}-{flags_id(flags)}-{fmt}-g{G}')


@pytest.mark.parametrize('in_fmt,xb,flags,fmt,G', list(_requant_cases()))
def test_requant_matches_reference(oracle, in_fmt, xb, flags, fmt, G):
    """Already quantized input (FP8 / FP4 + scales in each layout) cast again per token."""
    store = golden('requant')
    col, rnd, ue = flags
    key_in = f'{in_fmt}/{xb}/{flags_id(flags)}'
    q, qsf = golden_tensor(store, key_in + '/q'), golden_tensor(store, key_in + '/qsf')
    # the first cast of the chain is an ordinary cast: check it too
    x = golden_tensor(store, 'x')
    q0, qsf0 = oracle.cast(x, in_fmt, (xb, xb), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    assert_equal(q0, q)
    assert_equal(qsf0, qsf)
    out, sf = oracle.cast((q, qsf), fmt, (1, G), x_block_size=(xb, xb), round_sf=rnd, use_tma_aligned_col_major_sf=col,
                          use_packed_ue8m0=ue)
    assert_equal(out, golden_tensor(store, f'{key_in}/{fmt}/g{G}/out'))
    assert_equal(sf, golden_tensor(store, f'{key_in}/{fmt}/g{G}/sf'))


@pytest.mark.parametrize('gather', [False, True])
@pytest.mark.parametrize('src', ['bf16', 'fp8'])
@pytest.mark.parametrize('rnd', [False, True])
def test_per_channel_cast_fused_matches_reference(oracle, rnd, src, gather):
    store = golden('requant')
    x = golden_tensor(store, 'pc/x') if src == 'bf16' else (golden_tensor(store, 'pc/q8'), golden_tensor(store, 'pc/s8'))
    pos = golden_tensor(store, 'pc/pos') if gather else None
    out, sf = oracle.per_channel_cast_fused(x, 128, None if src == 'bf16' else 128, rnd, pos)
    assert_equal(out, golden_tensor(store, f'pc/{src}/r{int(rnd)}/g{int(gather)}/out'))
    assert_equal(sf, golden_tensor(store, f'pc/{src}/r{int(rnd)}/g{int(gather)}/sf'))


CONFIG_OPS = {
    'cfg1_per_token_e4m3_g128': ('cfg1', lambda o, x: o.cast(x, 'e4m3', (1, 128))),
    'cfg1_per_token_e4m3_g128_round': ('cfg1', lambda o, x: o.cast(x, 'e4m3', (1, 128), round_sf=True)),
    'cfg2_per_block_128x128': ('cfg2', lambda o, x: o.cast(x, 'e4m3', (128, 128))),
    'cfg2_per_channel_128': ('cfg2', lambda o, x: o.cast(x, 'e4m3', (128, 1))),
    'cfg4_fp4_g32_ue8m0': ('cfg4', lambda o, x: o.cast(x, 'e2m1', (1, 32), round_sf=True, use_tma_aligned_col_major_sf=True,
                                                       use_packed_ue8m0=True)),
    'cfg4_e5m6': ('cfg4', lambda o, x: o.cast_to_e5m6(x, x.shape[1])),
    'cfg5_per_token_e4m3_g128_ue8m0': ('cfg5', lambda o, x: o.cast(x, 'e4m3', (1, 128), round_sf=True,
                                                                   use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)),
}


def _sha(t: torch.Tensor) -> str:
    dense = torch.empty(t.shape, dtype=t.dtype)
    dense.copy_(t)
    return hashlib.sha256(dense.flatten().view(torch.uint8).numpy().tobytes()).hexdigest()


@pytest.mark.parametrize('name', sorted(CONFIG_OPS))
def test_benchmark_workloads_match_reference_digests(oracle, name):
    """Reduced-row versions of the benchmark workloads: the oracle's outputs hash to what the reference produced."""
    with open(os.path.join(GOLDEN, 'config_digests.json')) as f:
        want = json.load(f)[name]
    cfg, op = CONFIG_OPS[name]
    x = make_config_input(cfg, want['rows'])
    assert _sha(x) == want['x'], 'seeded input differs from the one the fixture was made with (torch RNG changed?)'
    out, sf = op(oracle, x)
    assert _sha(out) == want['out']
    assert _sha(sf) == want['sf']
    assert list(sf.shape) == want['sf_meta']['shape']


def test_swiglu_cast_on_benchmark_workload_close_to_reference(oracle):
    """The oracle against the reference on the benchmark workload of the fused SwiGLU cast (cfg3) at 1024 rows:
    2.1 M activations, 16384 scale groups of 128, default flags (fp32 scales).  The rule: scales identical, codes at most
    one step apart on at most 1e-4 of the elements, dequantised values of equal codes within 1e-3.

    fp32 scales cannot all be identical: a scale is max|y| / 448, so it moves with the last bit of the largest
    activation, and torch's CPU exp and this project's exp each miss the correctly rounded result for about 1-2 % of
    the bf16 arguments, on different arguments.  The count is asserted here, not hidden: 14 of 16384 scales differ,
    by at most 2 ulp, and no code differs at all."""
    from helpers import swiglu_cast_differences
    from tilekernels_b200.testing import make_config_input
    import hashlib
    store = golden('swiglu_cfg3')
    x = make_config_input('cfg3', 1024)
    assert hashlib.sha256(x.view(torch.uint8).numpy().tobytes()).hexdigest() == str(store['x1024.sha256'])
    out, sf = oracle.cast(oracle.swiglu_forward(x), 'e4m3', (1, 128))
    d = swiglu_cast_differences(out, sf, golden_tensor(store, 'plain/000/out'), golden_tensor(store, 'plain/000/sf'), 128,
                                oracle.sf_to_float)
    assert d['scales'] == 16384 and d['scales_differing'] == 14 and d['scale_max_ulp'] <= 2, d
    assert d['code_max_step'] <= 1 and d['codes_differing'] <= 1e-4 * d['codes'], d
    assert d['codes_differing'] == 0, d
    assert d['dequant_max_rel_equal_codes'] <= 1e-3, d


def test_swiglu_cast_on_benchmark_workload_pow2_scales_identical(oracle):
    """Same workload, 512 rows, power-of-two scales in the packed ue8m0 layout: scales, strides and codes all
    identical to the reference."""
    from tilekernels_b200.testing import make_config_input
    store = golden('swiglu_cfg3')
    x = make_config_input('cfg3', 512)
    out, sf = oracle.cast(oracle.swiglu_forward(x), 'e4m3', (1, 128), round_sf=True, use_tma_aligned_col_major_sf=True,
                          use_packed_ue8m0=True)
    assert_equal(sf, golden_tensor(store, 'plain/111/sf'))
    assert_equal(out, golden_tensor(store, 'plain/111/out'))


@pytest.mark.parametrize('flags', ['000', '111'])
def test_swiglu_cast_on_benchmark_workload_weights_and_clamp(oracle, flags):
    """256 rows of the workload with row weights, clamp 2.5 and clamp counters."""
    from helpers import swiglu_cast_differences
    from tilekernels_b200.testing import make_config_input
    store = golden('swiglu_cfg3')
    x = make_config_input('cfg3', 256)
    counts = torch.zeros(3, dtype=torch.int64)
    y = oracle.swiglu_forward(x, golden_tensor(store, 'moe/pos_to_token_topk'), golden_tensor(store, 'moe/topk_weights'), 2.5, counts)
    assert torch.equal(counts, golden_tensor(store, 'moe/counts'))
    col = rnd = ue = flags == '111'
    out, sf = oracle.cast(y, 'e4m3', (1, 128), round_sf=rnd, use_tma_aligned_col_major_sf=col, use_packed_ue8m0=ue)
    out_ref, sf_ref = golden_tensor(store, f'moe/{flags}/out'), golden_tensor(store, f'moe/{flags}/sf')
    d = swiglu_cast_differences(out, sf, out_ref, sf_ref, 128, oracle.sf_to_float)
    if rnd:
        assert_equal(sf, sf_ref)
    else:
        assert d['scales_differing'] <= 4 and d['scale_max_ulp'] <= 2, d
    assert d['code_max_step'] <= 1 and d['codes_differing'] <= 1e-4 * d['codes'], d
    assert d['dequant_max_rel_equal_codes'] <= 1e-3, d
