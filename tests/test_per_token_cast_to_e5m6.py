"""per_token_cast(..., 'e5m6', hidden) on the GPU against the oracle
(parametrised as the reference's tests/quant/test_per_token_cast_to_e5m6.py:38-83)."""
import pytest
import torch

from helpers import FLAG_SETS, flags_id, to_host
from tilekernels_b200.testing import assert_equal, generate_e5m6_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('flags', FLAG_SETS, ids=flags_id)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32], ids=['bf16', 'fp32'])
@pytest.mark.parametrize('num_tokens,hidden', [(4001, 576), (4001, 7168), (513, 2048), (130, 2560), (65, 3072), (33, 4096), (17, 6144),
                                               (5, 8), (7, 40), (3, 16384), (2, 40960)])
def test_per_token_cast_to_e5m6(oracle, cuda_device, num_tokens, hidden, dtype, flags):
    from tilekernels_b200 import quant
    col, rnd, ue = flags
    g = torch.Generator().manual_seed(hidden + num_tokens)
    for x, _special in generate_e5m6_inputs(num_tokens, hidden, dtype, device='cpu', generator=g):
        out, sf = quant.per_token_cast(x.to(cuda_device), 'e5m6', hidden, use_tma_aligned_col_major_sf=col, round_sf=rnd,
                                       use_packed_ue8m0=ue)
        out_ref, sf_ref = oracle.cast_to_e5m6(x, hidden, col, rnd, ue)
        assert_equal(to_host(out), out_ref)
        assert_equal(to_host(sf), sf_ref)


def test_e5m6_strided_rows(oracle, cuda_device):
    from tilekernels_b200 import quant
    g = torch.Generator().manual_seed(11)
    base = torch.randn((300, 4096), generator=g).to(torch.bfloat16)
    out, sf = quant.per_token_cast_to_e5m6(base.to(cuda_device)[:, :2048], 2048, round_sf=True)
    out_ref, sf_ref = oracle.cast_to_e5m6(base[:, :2048], 2048, False, True, False)
    assert_equal(to_host(out), out_ref)
    assert_equal(to_host(sf), sf_ref)
