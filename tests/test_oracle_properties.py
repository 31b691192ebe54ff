"""Size-independent properties of the CPU oracle on random shapes (hypothesis): what the GPU suite checks at full
size, checked here on many small ragged cases."""
import torch
from hypothesis import given, settings, strategies as st

FORMATS = {'e4m3': 448.0, 'e2m1': 6.0}


@st.composite
def cast_case(draw):
    fmt = draw(st.sampled_from(sorted(FORMATS)))
    group = draw(st.sampled_from((16, 32, 64, 128)))
    tokens = draw(st.integers(1, 24))
    hidden = 16 * draw(st.integers(1, 24))
    seed = draw(st.integers(0, 2**31 - 1))
    magnitude = draw(st.sampled_from((1e-3, 1.0, 300.0)))
    round_sf = draw(st.booleans())
    return fmt, group, tokens, hidden, seed, magnitude, round_sf


@settings(max_examples=30, deadline=None)
@given(cast_case())
def test_dequantised_values_are_close_and_requantise_to_the_same_codes(oracle, case):
    fmt, group, tokens, hidden, seed, magnitude, round_sf = case
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn((tokens, hidden), generator=gen) * magnitude).to(torch.bfloat16)
    q, sf = oracle.cast(x, fmt, (1, group), round_sf=round_sf)
    back = oracle.cast_back((q, sf), 'fp32', (1, group))
    scale = oracle.sf_to_float(sf).repeat_interleave(group, dim=1)[:, :hidden]
    # half a step of the coarsest binade: 2^-4 of the maximum for e4m3 (3 mantissa bits), 2^-2 for e2m1 (1 bit)
    step = FORMATS[fmt] * scale * (2.0 ** -4 if fmt == 'e4m3' else 2.0 ** -2)
    assert bool(((back - x.float()).abs() <= step * 1.0001 + 1e-30).all())
    assert bool((back.abs() <= FORMATS[fmt] * scale * 1.0001).all())
    # idempotence: the dequantised tensor has the same group maxima or smaller, and casting it with the stored
    # scales gives back the same codes
    again = oracle.cast(back, fmt, (1, group), sf=oracle.sf_to_float(sf).contiguous())
    assert torch.equal(again.view(torch.uint8), q.view(torch.uint8))


@settings(max_examples=20, deadline=None)
@given(st.integers(1, 16), st.integers(1, 12), st.integers(0, 2**31 - 1))
def test_rows_are_independent(oracle, tokens, chunks, seed):
    """Per-token casts never look across rows: casting a row subset gives the same bytes (the property that lets
    the token dimension be split over GPUs with no exchange)."""
    hidden = 128 * chunks
    x = torch.randn((tokens, hidden), generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
    q, sf = oracle.cast(x, 'e4m3', (1, 128), round_sf=True)
    pick = torch.arange(0, tokens, 2)
    q2, sf2 = oracle.cast(x[pick].contiguous(), 'e4m3', (1, 128), round_sf=True)
    assert torch.equal(q2.view(torch.uint8), q[pick].view(torch.uint8))
    assert torch.equal(oracle.sf_to_float(sf2), oracle.sf_to_float(sf)[pick])
