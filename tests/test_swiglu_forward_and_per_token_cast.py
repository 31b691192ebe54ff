"""swiglu_forward_and_per_token_cast on the GPU against the oracle, bit for bit (the oracle and the kernel
share one exp routine).  Parametrised after the reference's
tests/quant/test_swiglu_forward_and_per_token_cast.py:34-133: weights on/off, pos_to_expert masking on/off,
group 128 or hidden, clamp None / 10 / 0.5 with exact clamp counters, two SM counts."""
import pytest
import torch

from helpers import flags_id, to_host
from tilekernels_b200.testing import assert_equal

pytestmark = pytest.mark.gpu


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
    for num_sms in (sm_total - 20, sm_total):
        config.set_num_sms(num_sms)
        counts = torch.zeros(3, dtype=torch.int64, device=cuda_device) if count else None
        out, sf = quant.swiglu_forward_and_per_token_cast(
            x, 'e4m3', g,
            pos_to_token_topk=pos_to_token_topk.to(cuda_device) if weighted else None,
            topk_weights=weights.to(cuda_device) if weighted else None,
            pos_to_expert=pos_to_expert.to(cuda_device) if masked else None,
            use_tma_aligned_col_major_sf=col, round_sf=rnd, use_packed_ue8m0=ue,
            swiglu_clamp_value=clamp, clamped_count=counts)
        # skipped rows are left unwritten by the kernel: blank them on both sides before comparing
        out_h = to_host(out).view(torch.uint8).masked_fill(mask, 0)
        assert torch.equal(out_h, out_ref.view(torch.uint8).masked_fill(mask, 0))
        sf_h, sf_r = to_host(sf).clone(), sf_ref.clone()
        sf_h[mask.expand_as(sf_h)] = 0
        sf_r[mask.expand_as(sf_r)] = 0
        assert_equal(sf_h, sf_r)
        if count:
            assert torch.equal(counts.cpu(), counts_ref)


def test_custom_sf_clamp_min(oracle, cuda_device):
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(3)
    x_cpu = (torch.randn((130, 512), generator=gen) * 1e-3).to(torch.bfloat16)
    out, sf = quant.swiglu_forward_and_per_token_cast(x_cpu.to(cuda_device), 'e4m3', 128, sf_clamp_min=1e-2)
    out_ref, sf_ref = oracle.cast(oracle.swiglu_forward(x_cpu), 'e4m3', (1, 128), clamp_min=1e-2)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)


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
