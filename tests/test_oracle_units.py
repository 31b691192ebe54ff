"""Element-level checks of the CPU oracle that need no fixture: its e4m3 converter against torch's own
float8 conversion, its exp() against float64, and the scale-factor layouts."""
import torch

from tilekernels_b200.testing import assert_equal


def test_e4m3_converter_matches_torch(oracle):
    g = torch.Generator().manual_seed(1)
    v = torch.cat([torch.randn(500000, generator=g) * s for s in (1e-3, 0.02, 1.0, 30.0, 400.0)] +
                  [torch.linspace(-470, 470, 200001), torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10])])
    want = v.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(oracle.convert_array(v, 'e4m3'), want)
    # every midpoint between neighbouring e4m3 values, and its float neighbours (ties must go to even)
    codes = torch.arange(0, 0x7E, dtype=torch.uint8)
    lo, hi = codes.view(torch.float8_e4m3fn).float(), (codes + 1).view(torch.float8_e4m3fn).float()
    mid = (lo + hi) / 2
    pts = torch.cat([mid, torch.nextafter(mid, hi), torch.nextafter(mid, lo)])
    pts = torch.cat([pts, -pts])
    assert torch.equal(oracle.convert_array(pts, 'e4m3'), pts.to(torch.float8_e4m3fn).view(torch.uint8))


def test_exp_is_within_one_ulp(oracle):
    x = torch.cat([torch.linspace(-87, 88, 2000001), torch.randn(1000000) * 3])
    y = oracle.expf(x).double()
    t = torch.exp(x.double())
    ulp = (y - t).abs() / torch.exp2(torch.floor(torch.log2(t)) - 23)
    assert ulp.max().item() < 1.0
    assert (y.float() == t.float()).float().mean().item() > 0.94
    # outside the clamp range only 1 + exp(x) is used: it must still be exact at the low end
    assert torch.all(1.0 + oracle.expf(torch.tensor([-87.0, -100.0, -1e30])) == 1.0)


def test_scale_layouts(oracle):
    # 6 tokens x 9 groups of 32: row-major, column-major (token pitch padded to 4) and packed ue8m0 (3 words per token)
    g = torch.Generator().manual_seed(2)
    x = torch.randn((6, 288), generator=g).to(torch.bfloat16)
    _, sf = oracle.cast(x, 'e4m3', (1, 32), round_sf=True)
    _, sf_col = oracle.cast(x, 'e4m3', (1, 32), round_sf=True, use_tma_aligned_col_major_sf=True)
    _, sf_pk = oracle.cast(x, 'e4m3', (1, 32), round_sf=True, use_tma_aligned_col_major_sf=True, use_packed_ue8m0=True)
    assert sf.shape == (6, 9) and sf.stride() == (9, 1)
    assert sf_col.shape == (6, 9) and sf_col.stride() == (1, 8) and torch.equal(sf_col, sf)
    assert sf_pk.shape == (6, 3) and sf_pk.stride() == (1, 8) and sf_pk.dtype == torch.int32
    exps = (sf.view(torch.int32) >> 23).to(torch.uint8)
    padded = torch.zeros((6, 12), dtype=torch.uint8)
    padded[:, :9] = exps
    assert_equal(sf_pk.contiguous(), padded.view(torch.int32))
    assert torch.equal(oracle.sf_to_float(sf_pk)[:, :9], sf)


def test_power_of_two_scale_shortcut_equals_division():
    """The kernels obtain a rounded scale's exponent as ((bits(amax) + C) >> 23) - p instead of dividing by the
    format maximum; the two agree for every amax at or above the clamp (exhaustive in C during development,
    sampled here across all exponents and around every mantissa boundary)."""
    for max_q, carry, p, clamp in ((448.0, 0x1FFFFF, 8, 1e-4), (6.0, 0x3FFFFF, 2, 6.0 * 2.0 ** -126), (65024.0, 0x01FFFF, 15, 1e-4)):
        lo = torch.tensor(clamp, dtype=torch.float32).view(torch.int32).item()
        g = torch.Generator().manual_seed(3)
        bits = torch.randint(lo, 0x7F7FFFFF, (4000000,), generator=g, dtype=torch.int64)
        edges = (torch.arange(1, 255, dtype=torch.int64) << 23).unsqueeze(1) + (0x800000 - carry - 1) + torch.arange(-3, 4)
        bits = torch.cat([bits, edges.flatten()[(edges.flatten() >= lo)]]).to(torch.int32)
        a = bits.view(torch.float32)
        sf = (a / torch.tensor(max_q, dtype=torch.float32)).view(torch.int32)
        want = ((sf - 1) >> 23) + 1
        got = ((bits.to(torch.int64) + carry) >> 23) - p
        assert torch.equal(want.to(torch.int64), got)


def test_swiglu_backward_agrees_with_double_precision(oracle):
    """The backward restatement against the same formulas evaluated in float64 (an independent check of the
    formulas, next to the reference fixtures): values within 1e-5 relative to the row's largest magnitude, the
    zeroing of clamped gradients exact, weight_grad within 1e-5 relative."""
    gen = torch.Generator().manual_seed(99)
    rows, hidden, G = 16, 256, 128
    x = (torch.randn((rows, 2 * hidden), generator=gen) * 2).to(torch.bfloat16)
    q, sf = oracle.cast(x, 'e4m3', (1, G))
    d = torch.randn((rows, hidden), generator=gen).to(torch.bfloat16)
    w = torch.rand((rows, 1), generator=gen)
    pos = torch.arange(rows, dtype=torch.int32)
    pos[3] = -1
    t2p = torch.arange(rows, dtype=torch.int32).view(rows, 1).clone()
    t2p[3] = -1
    for clamp in (None, 0.75):
        out, x_grad, w_grad = oracle.swiglu_backward((q, sf), d, w, pos, t2p, G, clamp)
        xf = oracle.cast_back((q, sf), 'fp32', (1, G)).double()
        g, u = xf[:, :hidden].clone(), xf[:, hidden:].clone()
        cg = torch.zeros_like(g, dtype=torch.bool)
        cu = torch.zeros_like(u, dtype=torch.bool)
        if clamp is not None:
            cg, cu = g > clamp, u.abs() > clamp
            g, u = g.clamp(max=clamp), u.clamp(-clamp, clamp)
        wr = w.double().flatten().clone()
        wr[3] = 0
        s = torch.sigmoid(g)
        act = g * s * u
        dd = d.double()
        q_ = dd * wr[:, None] * s
        dg = torch.where(cg, torch.zeros_like(g), q_ * u * (1 + g * (1 - s)))
        du = torch.where(cu, torch.zeros_like(u), q_ * g)
        ref_out, ref_grad = act * wr[:, None], torch.cat([dg, du], dim=1)

        def close(a, b):
            scale = b.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
            return ((a.double() - b).abs() / scale).max().item() <= 1e-5

        assert close(out, ref_out) and close(x_grad, ref_grad)
        assert torch.equal(x_grad[:, :hidden][cg], torch.zeros(int(cg.sum())))
        assert torch.equal(x_grad[:, hidden:][cu], torch.zeros(int(cu.sum())))
        ref_w = (dd * act).sum(dim=1)
        ref_w[3] = 0
        torch.testing.assert_close(w_grad.flatten().double(), ref_w, rtol=1e-5, atol=1e-5)
