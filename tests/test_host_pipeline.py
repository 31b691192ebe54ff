"""The host-buffer pipeline gives the bytes of the device-resident entry point, for every scale layout,
with row counts that do and do not divide into chunks."""
import pytest
import torch

from helpers import to_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('fmt,g,col,ue', [('e4m3', 128, True, True), ('e4m3', 128, False, False), ('e4m3', 64, True, False),
                                          ('e2m1', 32, True, True)])
@pytest.mark.parametrize('rows', [4096, 5000, 1024])
def test_host_pipeline_matches_device_api(cuda_device, fmt, g, col, ue, rows):
    from tilekernels_b200 import host, quant
    hidden = 1024
    gen = torch.Generator().manual_seed(rows)
    x = torch.randn((rows, hidden), generator=gen).to(torch.bfloat16).pin_memory()
    groups = hidden // g
    out = torch.empty((rows, hidden if fmt == 'e4m3' else hidden // 2), dtype=torch.uint8).pin_memory()
    if ue:
        sf = torch.empty((groups // 4, rows), dtype=torch.int32).pin_memory()
    elif col:
        sf = torch.empty((groups, rows), dtype=torch.float32).pin_memory()
    else:
        sf = torch.empty((rows, groups), dtype=torch.float32).pin_memory()
    pipe = host.HostCastPipeline(cuda_device, hidden=hidden, max_rows=8192, chunk_rows=2048, depth=2)
    for _ in range(2):  # the second call reuses the staging ring
        out_h, sf_h = pipe.per_token_cast_host(x, fmt, g, out, sf, use_tma_aligned_col_major_sf=col, round_sf=True,
                                               use_packed_ue8m0=ue)
        torch.cuda.synchronize()
        ref_out, ref_sf = quant.per_token_cast(x.to(cuda_device), fmt, g, None, col, True, ue)
        assert torch.equal(out_h, ref_out.view(torch.uint8).cpu())
        ref_sf = to_host(ref_sf)
        assert sf_h.shape == ref_sf.shape and sf_h.dtype == ref_sf.dtype
        assert torch.equal(sf_h, ref_sf)
