"""swiglu_backward_and_per_token_cast: the oracle against reference fixtures (CPU) and the CUDA kernel against the
oracle (GPU), following the reference's tests/quant/test_swiglu_backward_and_per_token_cast.py:57-103."""
import pytest
import torch

from helpers import golden, golden_tensor, to_host
from tilekernels_b200.testing import assert_equal

CLAMPS = (None, 10.0, 0.5)


def _ulp(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (a.contiguous().view(torch.int16 if a.dtype == torch.bfloat16 else torch.int32).to(torch.int64) -
            b.contiguous().view(torch.int16 if b.dtype == torch.bfloat16 else torch.int32).to(torch.int64)).abs()


@pytest.mark.parametrize('G', (32, 128))
@pytest.mark.parametrize('clamp', CLAMPS)
def test_oracle_close_to_reference(oracle, G, clamp):
    """The oracle and the reference differ in exp() only (torch's CPU routine against the FMA-only routine this
    project shares between oracle and kernel, both within 1 ulp).  Tolerances: bf16 results equal or one bf16 step
    apart on at most 1e-3 of the elements; power-of-two scales identical, fp32 scales within 16 ulp (1 - s
    cancels for saturated gates, which multiplies the 1-ulp difference); FP8 codes at most one apart on at most
    3e-3 of the elements; weight_grad within atol = rtol = 1e-4, the reference's own bound.  For gates below -87
    the shared exp clamps its argument (exp(88) instead of infinity), which leaves values of magnitude below
    1e-30 where the reference has a signed zero: those are compared by absolute difference."""
    store = golden('swiglu_backward')
    x = (golden_tensor(store, f'g{G}/q'), golden_tensor(store, f'g{G}/qsf'))
    d, w = golden_tensor(store, 'grad_out'), golden_tensor(store, 'weight')
    pos, t2p = golden_tensor(store, 'pos_to_token_topk'), golden_tensor(store, 'token_topk_to_pos')
    out, x_grad, w_grad = oracle.swiglu_backward(x, d, w, pos, t2p, G, clamp)
    key = f'g{G}/c{clamp}'
    for mine, ref in ((out.bfloat16(), golden_tensor(store, key + '/out')), (x_grad.bfloat16(), golden_tensor(store, key + '/x_grad'))):
        diff = _ulp(mine, ref)
        diff[(mine.float() - ref.float()).abs() <= 1e-30] = 0
        assert diff.max().item() <= 1 and (diff > 0).float().mean().item() <= 1e-3
    torch.testing.assert_close(w_grad, golden_tensor(store, key + '/weight_grad'), atol=1e-4, rtol=1e-4)
    for rnd in (False, True):
        fp8, sf = oracle.cast(x_grad, 'e4m3', (1, G), round_sf=rnd)
        fp8_ref, sf_ref = golden_tensor(store, f'{key}/r{int(rnd)}/fp8'), golden_tensor(store, f'{key}/r{int(rnd)}/sf')
        if rnd:
            assert_equal(sf, sf_ref)
        else:
            assert _ulp(sf, sf_ref).max().item() <= 16
        diff = (fp8.view(torch.uint8).to(torch.int32) - fp8_ref.view(torch.uint8).to(torch.int32)).abs()
        assert diff.max().item() <= 1 and (diff > 0).float().mean().item() <= 3e-3


def _routing(num_tokens: int, num_topk: int, num_pad: int, gen: torch.Generator):
    """A consistent pair of maps as tile_kernels.moe.get_fused_mapping produces them: some (token, k) pairs are
    unrouted (-1), the routed ones sit at distinct expanded positions, num_pad positions are padding (-1)."""
    entries = num_tokens * num_topk
    routed = torch.rand(entries, generator=gen) > 0.2
    num_routed = int(routed.sum().item())
    num_expand = num_routed + num_pad
    positions = torch.randperm(num_expand, generator=gen)[:num_routed].to(torch.int32)
    token_topk_to_pos = torch.full((entries,), -1, dtype=torch.int32)
    token_topk_to_pos[routed] = positions
    pos_to_token_topk = torch.full((num_expand,), -1, dtype=torch.int32)
    pos_to_token_topk[positions.long()] = torch.nonzero(routed).flatten().to(torch.int32)
    return pos_to_token_topk, token_topk_to_pos.view(num_tokens, num_topk)


def _params():
    for num_tokens, num_topk, num_pad in ((1, 1, 0), (37, 2, 5), (301, 6, 64), (1024, 8, 100)):
        for hidden in (256, 384, 1024, 2048, 3584):
            if num_tokens == 1024 and hidden not in (2048,):
                continue
            for G in (32, 128):
                for round_sf in (False, True):
                    for clamp in CLAMPS:
                        yield pytest.param(num_tokens, num_topk, num_pad, hidden, G, round_sf, clamp,
                                           id=f't{num_tokens}-k{num_topk}-h{hidden}-g{G}-r{int(round_sf)}-c{clamp}')


@pytest.mark.gpu
@pytest.mark.parametrize('num_tokens,num_topk,num_pad,hidden,G,round_sf,clamp', list(_params()))
def test_swiglu_backward_and_per_token_cast(oracle, cuda_device, num_tokens, num_topk, num_pad, hidden, G, round_sf, clamp):
    """Everything but weight_grad is bit-exact against the oracle.  weight_grad is a sum of `hidden` fp32 products
    whose order differs: it must lie within 2e-6 * sum(|grad_out * act|) of the oracle's double-precision sum (the
    reference's test allows atol = rtol = 1e-4 on unit-variance data)."""
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(num_tokens * 7 + hidden + G)
    pos, t2p = _routing(num_tokens, num_topk, num_pad, gen)
    rows = pos.numel()
    xb = (torch.randn((rows, 2 * hidden), generator=gen) * 2).to(torch.bfloat16)
    if rows > 3:
        xb[1] = 0
        xb[2] *= 30
    q, qsf = oracle.cast(xb, 'e4m3', (1, G))
    d = torch.randn((rows, hidden), generator=gen).to(torch.bfloat16)
    w = torch.rand((num_tokens, num_topk), generator=gen)
    out, (fp8, sf), x_grad, w_grad = quant.swiglu_backward_and_per_token_cast(
        (q.to(cuda_device), qsf.to(cuda_device)), d.to(cuda_device), w.to(cuda_device), pos.to(cuda_device), t2p.to(cuda_device),
        G, round_sf, clamp)
    out_ref, x_grad_ref, w_grad_ref = oracle.swiglu_backward((q, qsf), d, w, pos, t2p, G, clamp)
    fp8_ref, sf_ref = oracle.cast(x_grad_ref, 'e4m3', (1, G), round_sf=round_sf)
    assert out.dtype == torch.bfloat16 and x_grad.dtype == torch.bfloat16 and w_grad.dtype == torch.float32
    assert_equal(to_host(out), out_ref.bfloat16())
    assert_equal(to_host(x_grad), x_grad_ref.bfloat16())
    assert_equal(to_host(sf), sf_ref)
    assert_equal(to_host(fp8), fp8_ref)
    if rows == 0:
        return  # nothing is launched, weight_grad stays uninitialised (reference wrapper :235)
    act = oracle.swiglu_backward((q, qsf), d, torch.ones_like(w), pos, t2p, G, clamp)[0]   # weight 1: out = act
    bound = torch.zeros(num_tokens * num_topk, dtype=torch.float64)
    routed = pos >= 0
    bound[pos[routed].long()] = (d.double() * act.double()).abs().sum(dim=1)[routed]
    err = (to_host(w_grad).double() - w_grad_ref.double()).abs().flatten()
    assert bool((err <= 2e-6 * bound + 1e-30).all()), (err.max().item(), bound.max().item())


@pytest.mark.gpu
def test_backward_3d_input_and_empty(oracle, cuda_device):
    """A (experts, tokens, 2 * hidden) input is flattened (reference wrapper :210-213); no expanded token launches
    nothing and returns empty tensors of the right shapes."""
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(5)
    pos, t2p = _routing(24, 2, 0, gen)
    if pos.numel() % 2:  # the 3-D view below needs an even number of rows: add one padding row
        pos, t2p = _routing(24, 2, 1, torch.Generator().manual_seed(5))
    rows = pos.numel()
    assert rows % 2 == 0
    hidden = 256
    xb = torch.randn((rows, 2 * hidden), generator=gen).to(torch.bfloat16)
    q, qsf = oracle.cast(xb, 'e4m3', (1, 128))
    d = torch.randn((rows, hidden), generator=gen).to(torch.bfloat16)
    w = torch.rand((24, 2), generator=gen)
    args = (d.to(cuda_device), w.to(cuda_device), pos.to(cuda_device), t2p.to(cuda_device), 128)
    flat = quant.swiglu_backward_and_per_token_cast((q.to(cuda_device), qsf.to(cuda_device)), *args)
    cube = quant.swiglu_backward_and_per_token_cast((q.to(cuda_device).view(2, rows // 2, 2 * hidden), qsf.to(cuda_device)), *args)
    assert_equal(to_host(flat[0]), to_host(cube[0]))
    assert_equal(to_host(flat[1][0]), to_host(cube[1][0]))
    assert_equal(to_host(flat[2]), to_host(cube[2]))

    e = torch.empty
    out, (fp8, sf), x_grad, w_grad = quant.swiglu_backward_and_per_token_cast(
        (e((0, 512), dtype=torch.float8_e4m3fn, device=cuda_device), e((0, 4), dtype=torch.float32, device=cuda_device)),
        e((0, 256), dtype=torch.bfloat16, device=cuda_device), w.to(cuda_device), e((0,), dtype=torch.int32, device=cuda_device),
        torch.full((24, 2), -1, dtype=torch.int32, device=cuda_device), 128)
    assert out.shape == (0, 256) and fp8.shape == (0, 512) and sf.shape == (0, 4) and x_grad.shape == (0, 512) and w_grad.shape == (24, 2)
