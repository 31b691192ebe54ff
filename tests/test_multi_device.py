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


def test_wrappers_follow_their_tensors(oracle, cuda_device):
    """Every wrapper launches on the device of its input, whichever device is current: the calls below are made with
    device 0 current and tensors on the LAST visible device (the same device when only one is visible)."""
    from tilekernels_b200 import moe, quant
    dev = torch.device('cuda', torch.cuda.device_count() - 1)
    gen = torch.Generator().manual_seed(14)
    kw = dict(use_tma_aligned_col_major_sf=True, round_sf=True, use_packed_ue8m0=True)
    x = torch.randn((256, 1024), generator=gen).to(torch.bfloat16)
    with torch.cuda.device(0):
        xd = x.to(dev)
        q, qsf = quant.per_block_cast(xd, 'e4m3', (128, 128), **kw)
        q_ref, qsf_ref = oracle.cast(x, 'e4m3', (128, 128), **kw)
        assert_equal(to_host(q), q_ref)
        # re-quantising cast, dequantisation
        out, sf = quant.per_token_cast((q, qsf), 'e4m3', 128, x_block_size=(128, 128), **kw)
        out_ref, sf_ref = oracle.cast((q_ref, qsf_ref), 'e4m3', (1, 128), x_block_size=(128, 128), **kw)
        assert_equal(to_host(out), out_ref)
        assert_equal(to_host(sf), sf_ref)
        back = quant.cast_back((q, qsf), 'bf16', (128, 128))
        assert_equal(to_host(back), oracle.cast_back((q_ref, qsf_ref), 'bf16', (128, 128)))
        # FP4 and its lossless re-blocking
        q4, q4sf = quant.per_token_cast(xd, 'e2m1', 32, None, False, True, False)
        q4_ref, q4sf_ref = oracle.cast(x, 'e2m1', (1, 32), round_sf=True)
        out, sf = quant.per_block_cast_lossless((q4, q4sf), 'e4m3', (1, 32), (128, 128), False, True, False)
        out_ref, sf_ref = oracle.per_block_cast_lossless((q4_ref, q4sf_ref), (1, 32), (128, 128), False, False)
        assert_equal(to_host(out), out_ref)
        assert_equal(to_host(sf), sf_ref)
        # per-channel casts
        out, sf = quant.per_channel_cast(xd, 'e4m3', 128)
        out_ref, sf_ref = oracle.cast(x, 'e4m3', (128, 1))
        assert_equal(to_host(out), out_ref)
        assert_equal(to_host(sf), sf_ref)
        # row expansion
        t2p = torch.arange(512, dtype=torch.int32).view(256, 2)
        p2e = torch.zeros(512, dtype=torch.int32)
        out = moe.expand_to_fused(xd, t2p.to(dev), p2e.to(dev))
        assert_equal(to_host(out), oracle.expand_to_fused(x, t2p, p2e))
        # SwiGLU backward
        qx, qxsf = oracle.cast(x, 'e4m3', (1, 128))
        d = torch.randn((256, 512), generator=gen).to(torch.bfloat16)
        w = torch.rand((256, 1), generator=gen)
        pos = torch.arange(256, dtype=torch.int32)
        got = quant.swiglu_backward_and_per_token_cast((qx.to(dev), qxsf.to(dev)), d.to(dev), w.to(dev), pos.to(dev), pos.view(256, 1).to(dev), 128,
                                                       True, None)
        want = oracle.swiglu_backward((qx, qxsf), d, w, pos, pos.view(256, 1), 128, None)
        assert_equal(to_host(got[0]), want[0].bfloat16())
        assert_equal(to_host(got[2]), want[1].bfloat16())
    with torch.cuda.device(dev):
        from tilekernels_b200 import _lib
        assert _lib.lib().tkq_device_error() == 0
