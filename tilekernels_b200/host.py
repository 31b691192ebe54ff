"""Per-token cast for callers whose tensors live in host memory.

`HostCastPipeline.per_token_cast_host` takes pinned host tensors, moves the rows through the GPU in chunks and
leaves the quantized data and scales in pinned host tensors.  Host->device copies, the cast kernels and
device->host copies run on three streams over a ring of preallocated device staging buffers, so the two PCIe
directions and the kernels overlap; per call nothing is allocated.  The kernels are the same ones
`tilekernels_b200.quant.per_token_cast` launches, called through the C ABI with pointers into the staging ring.
"""

import torch

from . import _lib
from .quant.common import DTYPE_TO_ENUM, FMT_TO_ENUM
from .utils import align, ceil_div


class HostCastPipeline:
    def __init__(self, device: torch.device, hidden: int, max_rows: int, chunk_rows: int = 4096, depth: int = 3,
                 in_dtype: torch.dtype = torch.bfloat16):
        assert hidden % 16 == 0 and depth >= 2
        self.device = torch.device(device)
        self.hidden = hidden
        self.max_rows = max_rows
        self.chunk_rows = min(chunk_rows, max_rows)
        self.depth = depth
        self.in_dtype = in_dtype
        with torch.cuda.device(self.device):
            self.x_dev = [torch.empty((self.chunk_rows, hidden), dtype=in_dtype, device=self.device) for _ in range(depth)]
            self.out_dev = [torch.empty((self.chunk_rows, hidden), dtype=torch.uint8, device=self.device) for _ in range(depth)]
            # scales of the whole tensor stay on the device until the end of a call (1/128 of the data or less)
            self.sf_dev = torch.empty(ceil_div(hidden, 16) * align(max_rows, 4) * 4, dtype=torch.uint8, device=self.device)
            self.h2d = torch.cuda.Stream(self.device)
            self.compute = torch.cuda.Stream(self.device)
            self.d2h = torch.cuda.Stream(self.device)
            self.ev_loaded = [torch.cuda.Event() for _ in range(depth)]
            self.ev_cast = [torch.cuda.Event() for _ in range(depth)]
            self.ev_free = [torch.cuda.Event() for _ in range(depth)]

    def per_token_cast_host(self, x: torch.Tensor, fmt: str, num_per_channels: int, out: torch.Tensor, out_sf: torch.Tensor,
                            use_tma_aligned_col_major_sf: bool = True, round_sf: bool = True,
                            use_packed_ue8m0: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
        """Cast pinned host `x` (num_tokens, hidden) into pinned host `out` and `out_sf`.

        out     e4m3: (num_tokens, hidden) float8_e4m3fn or uint8; e2m1: (num_tokens, hidden / 2) int8 or uint8
        out_sf  contiguous scale *storage*: row-major fp32 (num_tokens, groups); column-major fp32 (groups, num_tokens);
                packed ue8m0 int32 (ceil(groups / 4), num_tokens).  num_tokens must be a multiple of 4 for the
                column-major layouts (then the storage has no padding).
        Returns (out, scales) where scales is `out_sf` viewed as the reference returns it (transposed when
        column-major).  The work is ordered after the caller's current stream and that stream waits for it.
        """
        assert fmt in ('e4m3', 'e2m1') and num_per_channels in (16, 32, 64, 128)
        assert x.is_pinned() and out.is_pinned() and out_sf.is_pinned() and x.is_contiguous() and out.is_contiguous()
        assert x.dtype == self.in_dtype and x.dim() == 2 and x.shape[1] == self.hidden and x.shape[0] <= self.max_rows
        col_major, packed = use_tma_aligned_col_major_sf, use_packed_ue8m0
        assert col_major or not packed
        T, H = x.shape
        groups = ceil_div(H, num_per_channels)
        out_cols = H if fmt == 'e4m3' else H // 2
        assert tuple(out.shape) == (T, out_cols) and out.element_size() == 1
        if packed:
            sf_shape, sf_dtype, sf_stride = (ceil_div(groups, 4), T), torch.int32, 4 * T
        elif col_major:
            sf_shape, sf_dtype, sf_stride = (groups, T), torch.float32, T
        else:
            sf_shape, sf_dtype, sf_stride = (T, groups), torch.float32, groups
        assert not col_major or T % 4 == 0
        assert tuple(out_sf.shape) == sf_shape and out_sf.dtype == sf_dtype and out_sf.is_contiguous()
        flags = (_lib.ROUND_SF if round_sf else 0) | (_lib.SF_COL_MAJOR if col_major else 0) | (_lib.SF_UE8M0 if packed else 0)
        sf_bytes = out_sf.numel() * out_sf.element_size()
        sf_dev = self.sf_dev[:sf_bytes]
        lib = _lib.lib()

        caller = torch.cuda.current_stream(self.device)
        self.h2d.wait_stream(caller)
        self.d2h.wait_stream(caller)
        with torch.cuda.device(self.device):
            for i, r0 in enumerate(range(0, T, self.chunk_rows)):
                n = min(self.chunk_rows, T - r0)
                slot = i % self.depth
                with torch.cuda.stream(self.h2d):
                    if i >= self.depth:
                        self.h2d.wait_event(self.ev_free[slot])
                    self.x_dev[slot][:n].copy_(x[r0:r0 + n], non_blocking=True)
                    self.ev_loaded[slot].record(self.h2d)
                self.compute.wait_event(self.ev_loaded[slot])
                # scale pointer of this chunk inside the whole-tensor storage: rows advance along the fast axis
                # in the column-major layouts and along the slow axis in the row-major one
                sf_off = r0 * 4 if col_major else r0 * groups * 4
                rc = lib.tkq_per_token_cast(self.x_dev[slot].data_ptr(), DTYPE_TO_ENUM[self.in_dtype], n, H, H, FMT_TO_ENUM[fmt],
                                            num_per_channels, flags, self.out_dev[slot].data_ptr(), sf_dev.data_ptr() + sf_off,
                                            sf_stride, self.compute.cuda_stream)
                _lib.check(rc, 'tkq_per_token_cast')
                self.ev_cast[slot].record(self.compute)
                with torch.cuda.stream(self.d2h):
                    self.d2h.wait_event(self.ev_cast[slot])
                    out[r0:r0 + n].view(torch.uint8).copy_(self.out_dev[slot].view(-1)[:n * out_cols].view(n, out_cols), non_blocking=True)
                    self.ev_free[slot].record(self.d2h)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_stream(self.compute)
                out_sf.view(torch.uint8).view(-1).copy_(sf_dev, non_blocking=True)
        caller.wait_stream(self.d2h)
        return out, (out_sf.T if col_major else out_sf)
