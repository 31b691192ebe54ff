"""swiglu_forward_and_per_token_cast on the GPU against the oracle.  Parametrised after the reference's
tests/quant/test_swiglu_forward_and_per_token_cast.py:34-133: weights on/off, pos_to_expert masking on/off,
group 128 or hidden, clamp None / 10 / 0.5 with exact clamp counters, two SM counts.

Scales and clamp counters equal the oracle's bit for bit in every case.  The FP8 codes equal the oracle's bit
for bit when the exact evaluation is selected (config.set_exact_swiglu_codes) and wherever the library has no
approximate kernel (fp32 input, one scale per token, rows shorter than 1024); by default the bf16 / group-128
kernel derives them from hardware-approximate exp and reciprocal, and the rule is: at most one code apart, on at
most 1e-4 of the elements.  One element of a small tensor is already more than 1e-4 of it, so a case of fewer
than 10^6 elements may hold ONE such element and the rate is asserted over all cases together at the end."""
import pytest
import torch

from helpers import flags_id, to_host
from tilekernels_b200.testing import assert_equal

pytestmark = pytest.mark.gpu

_totals = {'codes': 0, 'differing': 0, 'cases': 0}


def _check_codes(out_h: torch.Tensor, out_ref: torch.Tensor, exact: bool) -> None:
    """out_h / out_ref: uint8 code tensors on the CPU."""
    if exact:
        assert torch.equal(out_h, out_ref)
        return
    diff = (out_h.to(torch.int32) - out_ref.to(torch.int32)).abs()
    differing = int((diff > 0).sum())
    assert differing == 0 or int(diff.max()) == 1, f'codes more than one step apart (max {int(diff.max())})'
    assert differing <= max(1, int(1e-4 * diff.numel())), f'{differing} of {diff.numel()} codes differ'
    _totals['codes'] += diff.numel()
    _totals['differing'] += differing
    _totals['cases'] += 1


def _routing(num_tokens, g):
    """A synthetic MoE layout: ~8% of the rows are padding (negative expert / position)."""
    pad = torch.rand(num_tokens, generator=g) < 0.08
    pos_to_expert = torch.randint(0, 8, (num_tokens,), generator=g, dtype=torch.int32)
    pos_to_expert[pad] = -1
    n_src, topk = max(1, num_tokens // 6), 6
    pos_to_token_topk = torch.randint(0, n_src * topk, (num_tokens,), generator=g, dtype=torch.int32)
    pos_to_token_topk[pad] = -1
    weights = torch.randn((n_src, topk), generator=g)
    return pos_to_expert, pos_to_token_topk, weights


def _params():
    for num_tokens, hidden in ((4001, 288 * 0 + 1024), (2050, 3584), (515, 2048), (33, 1280), (3, 128)):
        for dtype in (torch.bfloat16, torch.float32):
            for masked in (True, False):
                for weighted in (True, False):
                    for g in (128, hidden):
                        for flags in ((False, True, False), (True, True, True), (False, False, False)):
                            if (flags[2] and weighted) or (flags[0] and g == hidden):
                                continue
                            if dtype == torch.float32 and (num_tokens > 2050 or not flags[1]):
                                continue
                            for clamp in (None, 10.0, 0.5):
                                yield pytest.param(num_tokens, hidden, dtype, masked, weighted, g, flags, clamp,
                                                   id=f'{num_tokens}x{hidden}-{str(dtype)[6:]}-m{int(masked)}-w{int(weighted)}-g{g}-'
                                                      f'{flags_id(flags)}-c{clamp}')


@pytest.mark.parametrize('num_tokens,hidden,dtype,masked,weighted,g,flags,clamp', list(_params()))
def test_swiglu_forward_and_per_token_cast(oracle, cuda_device, num_tokens, hidden, dtype, masked, weighted, g, flags, clamp):
    from tilekernels_b200 import config, quant
    col, rnd, ue = flags
    gen = torch.Generator().manual_seed(num_tokens + hidden)
    x_cpu = (torch.randn((num_tokens, 2 * hidden), generator=gen) * 1.5).to(dtype)
    pos_to_expert, pos_to_token_topk, weights = _routing(num_tokens, gen)
    if masked:
        x_cpu[pos_to_expert < 0] = 0  # padding rows hold zeros after expansion, as in the reference's test data

    count = clamp is not None and g != hidden
    counts_ref = torch.zeros(3, dtype=torch.int64)
    y = oracle.swiglu_forward(x_cpu, pos_to_token_topk if weighted else None, weights if weighted else None, clamp,
                              counts_ref if count else None)
    mask = (pos_to_expert < 0).unsqueeze(-1) if masked else torch.zeros((num_tokens, 1), dtype=torch.bool)
    y = y.masked_fill(mask, 0)
    out_ref, sf_ref = oracle.cast(y, 'e4m3', (1, g), use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)

    x = x_cpu.to(cuda_device)
    sm_total = config.get_device_num_sms()
    for num_sms, exact in ((sm_total - 20, False), (sm_total, False), (sm_total, True)):
        config.set_num_sms(num_sms)
        config.set_exact_swiglu_codes(exact)
        counts = torch.zeros(3, dtype=torch.int64, device=cuda_device) if count else None
        out, sf = quant.swiglu_forward_and_per_token_cast(
            x, 'e4m3', g,
            pos_to_token_topk=pos_to_token_topk.to(cuda_device) if weighted else None,
            topk_weights=weights.to(cuda_device) if weighted else None,
            pos_to_expert=pos_to_expert.to(cuda_device) if masked else None,
            use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue,
            swiglu_clamp_value=clamp, clamped_count=counts)
        config.set_exact_swiglu_codes(False)
        # skipped rows are left unwritten by the kernel: blank them on both sides before comparing
        out_h = to_host(out).view(torch.uint8).masked_fill(mask, 0)
        approximate = not exact and dtype == torch.bfloat16 and g == 128 and hidden >= 1024
        _check_codes(out_h, out_ref.view(torch.uint8).masked_fill(mask, 0), exact=not approximate)
        sf_h, sf_r = to_host(sf).clone(), sf_ref.clone()
        sf_h[mask.expand_as(sf_h)] = 0
        sf_r[mask.expand_as(sf_r)] = 0
        assert_equal(sf_h, sf_r)
        if count:
            assert torch.equal(counts.cpu(), counts_ref)


@pytest.mark.parametrize('hidden', [512, 2048])
@pytest.mark.parametrize('clamp_min', [1e-2, 1e-20, 1e-35])
def test_custom_sf_clamp_min(oracle, cuda_device, hidden, clamp_min):
    """Custom clamps of the maximum, with rows small enough for the clamp to decide the scale.  A clamp below 1e-30
    takes the exact kernel (the approximate one needs every decisive value to be a normal number)."""
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(3)
    x_cpu = (torch.randn((130, 2 * hidden), generator=gen) * 1e-3).to(torch.bfloat16)
    x_cpu[5] *= 1e-12
    x_cpu[6] *= 1e-19
    x_cpu[7] = 0
    out, sf = quant.swiglu_forward_and_per_token_cast(x_cpu.to(cuda_device), 'e4m3', 128, sf_clamp_min=clamp_min)
    out_ref, sf_ref = oracle.cast(oracle.swiglu_forward(x_cpu), 'e4m3', (1, 128), clamp_min=clamp_min)
    assert_equal(to_host(sf), sf_ref)
    _check_codes(to_host(out).view(torch.uint8), out_ref.view(torch.uint8), exact=hidden < 1024 or clamp_min < 1e-30)


def _adversarial_input(gen, kind: str) -> torch.Tensor:
    """[256, 2 * 2048] bf16 inputs built to stress the choice of the exactly evaluated elements."""
    T, H = 256, 2048
    x = torch.randn((T, 2 * H), generator=gen)
    if kind == 'ties':
        # many equal or nearly equal (gate, up) pairs in every group: the two largest activations of a group are
        # often within a few ulp of each other, in different lanes and in the same lane
        base = torch.randn((T, H // 128, 1, 2), generator=gen).expand(T, H // 128, 128, 2) * 3
        jitter = (torch.rand((T, H // 128, 128, 2), generator=gen) < 0.9).float()
        pairs = base * (1 - jitter) + torch.randn((T, H // 128, 128, 2), generator=gen) * jitter
        x = torch.cat([pairs[..., 0].reshape(T, H), pairs[..., 1].reshape(T, H)], dim=1)
    elif kind == 'quantised':
        # gates and ups on a coarse grid: a few hundred distinct activations per row, so exact ties abound
        x = (x * 4).round() / 4
    elif kind == 'negative_gates':
        # gates between -100 and -60 (exp overflows or nearly so) next to ordinary ones, huge ups beside them
        x[:, :H] = torch.where(torch.rand((T, H), generator=gen) < 0.05, -60 - 40 * torch.rand((T, H), generator=gen), x[:, :H])
        x[:, H:] *= torch.where(torch.rand((T, H), generator=gen) < 0.02, 1e20, 1.0)
        x[3, :H] = -85.0
        x[4, :H] = -95.0
    elif kind == 'tiny':
        x[:, :H] *= 10.0 ** (-30 * torch.rand((T, 1), generator=gen))
        x[:, H:] *= 10.0 ** (-8 * torch.rand((T, 1), generator=gen))
        x[9] = 0
        x[10, :H] = 0
    elif kind == 'large':
        x[:, :H] *= 20
        x[:, H:] *= 1e4
    return x.to(torch.bfloat16)


@pytest.mark.parametrize('flags', [(False, False, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('clamp', [None, 7.0])
@pytest.mark.parametrize('kind', ['ties', 'quantised', 'negative_gates', 'tiny', 'large'])
def test_exact_scales_on_adversarial_inputs(oracle, cuda_device, kind, clamp, flags):
    """The approximate kernel's scales must equal the exactly evaluated ones whatever the data: near-ties between
    the largest activations of a group, gates where the hardware exp overflows, tiny and huge values."""
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    gen = torch.Generator().manual_seed(len(kind) * 7 + (clamp is not None))
    x_cpu = _adversarial_input(gen, kind)
    out, sf = quant.swiglu_forward_and_per_token_cast(x_cpu.to(cuda_device), 'e4m3', 128, use_tma_aligned_col_major_sf=col,
                                                      round_sf=rnd, use_packed_ue8m0=ue, swiglu_clamp_value=clamp)
    out_ref, sf_ref = oracle.cast(oracle.swiglu_forward(x_cpu, swiglu_clamp_value=clamp), 'e4m3', (1, 128),
                                  use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue)
    assert_equal(to_host(sf), sf_ref)
    diff = (to_host(out).view(torch.uint8).to(torch.int32) - out_ref.view(torch.uint8).to(torch.int32)).abs()
    # data built from few distinct values repeats whatever code an approximation moves, so only the step is bounded
    # here for those; the random kinds keep the 1e-4 rule
    assert int(diff.max()) <= 1
    if kind in ('negative_gates', 'tiny', 'large'):
        assert int((diff > 0).sum()) <= max(1, int(1e-4 * diff.numel()))


@pytest.mark.parametrize('clamp', [None, 10.0, 0.5, 0.3])
@pytest.mark.parametrize('round_sf', [False, True])
@pytest.mark.parametrize('without_transpose', [False, True])
@pytest.mark.parametrize('num_per_tokens', [32, 128])
@pytest.mark.parametrize('num_tokens,hidden', [(4096, 1024), (1024, 3584), (128, 64), (384, 1280)])
def test_swiglu_forward_and_per_channel_cast_and_transpose(oracle, cuda_device, num_tokens, hidden, num_per_tokens, without_transpose,
                                                           round_sf, clamp):
    """As the reference's tests/quant/test_swiglu_forward_and_per_channel_cast_and_transpose.py:44-85: the bf16-rounded
    activation is cast per (n x 1) block; data transposed unless without_transpose."""
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(num_tokens + hidden + num_per_tokens)
    x = (torch.randn((num_tokens, 2 * hidden), generator=gen) * 1.5).to(torch.bfloat16)
    x[7] = 0
    out, sf = quant.swiglu_forward_and_per_channel_cast_and_transpose(x.to(cuda_device), 'e4m3', num_per_tokens, round_sf,
                                                                        without_transpose, clamp)
    act = oracle.swiglu_forward(x, swiglu_clamp_value=clamp).bfloat16()
    out_ref, sf_ref = oracle.cast(act, 'e4m3', (num_per_tokens, 1), round_sf=round_sf)
    if not without_transpose:
        out_ref = out_ref.view(torch.uint8).T.contiguous().view(torch.float8_e4m3fn)
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(out), out_ref)


@pytest.mark.parametrize('flags', [(False, False, False), (True, True, True)], ids=flags_id)
@pytest.mark.parametrize('hidden', [1024, 1152, 2176, 4096, 7168, 16384])
def test_row_segments_of_the_staged_kernel(oracle, cuda_device, hidden, flags):
    """Rows longer and shorter than one 2048-activation segment, with full and partly filled last segments."""
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    gen = torch.Generator().manual_seed(hidden)
    x_cpu = (torch.randn((37, 2 * hidden), generator=gen) * 2).to(torch.bfloat16)
    out, sf = quant.swiglu_forward_and_per_token_cast(x_cpu.to(cuda_device), 'e4m3', 128, use_tma_aligned_col_major_sf=col,
                                                      round_sf=rnd, use_packed_ue8m0=ue)
    out_ref, sf_ref = oracle.cast(oracle.swiglu_forward(x_cpu), 'e4m3', (1, 128), use_tma_aligned_col_major_sf=col, round_sf=rnd,
                                  use_packed_ue8m0=ue)
    assert_equal(to_host(sf), sf_ref)
    _check_codes(to_host(out).view(torch.uint8), out_ref.view(torch.uint8), exact=False)


@pytest.mark.parametrize('seed', range(24))
def test_random_shapes_and_options_of_the_staged_kernel(oracle, cuda_device, seed):
    """Seeded random draws of everything the staged kernel depends on: tokens, hidden (any multiple of 128 from 1024),
    scale layout, clamp, counters, row weights, expert mask, input scale."""
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(1000 + seed)
    draw = lambda n: int(torch.randint(0, n, (1,), generator=gen))
    num_tokens = (1, 2, 7, 64, 129, 777, 1500)[draw(7)]
    hidden = 128 * (8 + draw(57))
    col, rnd, ue = ((False, False, False), (False, True, False), (True, True, False), (True, True, True))[draw(4)]
    clamp = (None, None, 10.0, 1.0, 0.25)[draw(5)]
    weighted, masked, count = draw(2) == 1 and not ue, draw(2) == 1, clamp is not None and draw(2) == 1
    x_cpu = (torch.randn((num_tokens, 2 * hidden), generator=gen) * (0.05, 1.0, 3.0, 20.0)[draw(4)]).to(torch.bfloat16)
    pos_to_expert, pos_to_token_topk, weights = _routing(num_tokens, gen)
    if masked:
        x_cpu[pos_to_expert < 0] = 0
    counts_ref = torch.zeros(3, dtype=torch.int64)
    y = oracle.swiglu_forward(x_cpu, pos_to_token_topk if weighted else None, weights if weighted else None, clamp,
                              counts_ref if count else None)
    mask = (pos_to_expert < 0).unsqueeze(-1) if masked else torch.zeros((num_tokens, 1), dtype=torch.bool)
    out_ref, sf_ref = oracle.cast(y.masked_fill(mask, 0), 'e4m3', (1, 128), use_tma_aligned_col_major_sf=col, round_sf=rnd,
                                  use_packed_ue8m0=ue)
    counts = torch.zeros(3, dtype=torch.int64, device=cuda_device) if count else None
    out, sf = quant.swiglu_forward_and_per_token_cast(
        x_cpu.to(cuda_device), 'e4m3', 128,
        pos_to_token_topk=pos_to_token_topk.to(cuda_device) if weighted else None,
        topk_weights=weights.to(cuda_device) if weighted else None,
        pos_to_expert=pos_to_expert.to(cuda_device) if masked else None,
        use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue, swiglu_clamp_value=clamp, clamped_count=counts)
    sf_h, sf_r = to_host(sf).clone(), sf_ref.clone()
    sf_h[mask.expand_as(sf_h)] = 0
    sf_r[mask.expand_as(sf_r)] = 0
    assert_equal(sf_h, sf_r)
    if count:
        # rows the mask skips are not counted by the kernel; the oracle saw them as zeros, which no clamp touches
        assert torch.equal(counts.cpu(), counts_ref)
    diff = (to_host(out).view(torch.uint8).masked_fill(mask, 0).to(torch.int32) -
            out_ref.view(torch.uint8).masked_fill(mask, 0).to(torch.int32)).abs()
    assert int(diff.max()) <= 1 and int((diff > 0).sum()) <= max(2, int(1e-4 * diff.numel()))


def test_zz_overall_code_difference_rate():
    """Over every approximate case of this file together (it runs last): far below the 1e-4 the rule allows."""
    if _totals['codes'] < 10 ** 7:
        pytest.skip('needs the parametrised cases of this file to have run in the same process')
    assert _totals['differing'] <= 1e-5 * _totals['codes'], _totals
