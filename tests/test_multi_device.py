"""One thread, several devices: the kernels that need a raised dynamic shared-memory limit (fp32 per-block cast,
E5M6 with long rows, the transposing per-channel cast) and the occupancy-sized grids must work on every visible
device in turn, because those settings belong to a (device, kernel) pair.  With one visible device the loop runs
once."""
import pytest
import torch

from helpers import to_host
from tilekernels_b200.testing import assert_equal

pytestmark = pytest.mark.gpu


def test_casts_on_every_visible_device(oracle, cuda_device):
    from tilekernels_b200 import quant
    gen = torch.Generator().manual_seed(12)
    x32 = torch.randn((256, 512), generator=gen)
    xlong = torch.randn((24, 16384), generator=gen).to(torch.bfloat16)
    xb = torch.randn((256, 256), generator=gen).to(torch.bfloat16)
    xs = torch.randn((64, 4096), generator=gen).to(torch.bfloat16)
    want_block = oracle.cast(x32, 'e4m3', (128, 128))
    want_e5m6 = oracle.cast_to_e5m6(xlong, xlong.shape[1])
    want_t = oracle.cast(xb, 'e4m3', (128, 1))
    want_sw = oracle.cast(oracle.swiglu_forward(xs), 'e4m3', (1, 128))
    order = list(range(torch.cuda.device_count()))
    for index in order + order[::-1]:      # forth and back: a cache keyed by the kernel alone would fail on the way
        dev = torch.device('cuda', index)
        out, sf = quant.per_block_cast(x32.to(dev), 'e4m3', (128, 128))
        assert_equal(to_host(out), want_block[0])
        assert_equal(to_host(sf), want_block[1])
        out, sf = quant.per_token_cast(xlong.to(dev), 'e5m6', xlong.shape[1])
        assert_equal(to_host(out), want_e5m6[0])
        assert_equal(to_host(sf), want_e5m6[1])
        out, sf = quant.per_channel_cast_and_transpose(xb.to(dev), 'e4m3', 128)
        assert_equal(to_host(sf), want_t[1])
        assert torch.equal(to_host(out).view(torch.uint8), want_t[0].view(torch.uint8).T.contiguous())
        out, sf = quant.swiglu_forward_and_per_token_cast(xs.to(dev), 'e4m3', 128)
        assert_equal(to_host(sf), want_sw[1])
        with torch.cuda.device(dev):
            from tilekernels_b200 import _lib
            assert _lib.lib().tkq_device_error() == 0
