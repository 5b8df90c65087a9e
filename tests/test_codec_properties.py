"""Properties of the storage codecs on generated tensors: quantising what a codec produced changes nothing (each codec
is a projection onto its own grid), the error of one pass is bounded by the format's step, nibble packing is lossless,
and the 128-point Hadamard used by EXL3 is its own inverse."""
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.quant import codecs as C

SHAPES = st.tuples(st.sampled_from([16, 32, 128]), st.sampled_from([128, 256]))
SCALES = st.sampled_from([1e-3, 0.02, 1.0, 37.0])


def _w(shape, scale, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(*shape, generator=g) * scale
    w[0, :7] = 0.0                                    # an all-zero stretch inside a group
    return w


@settings(max_examples=40, deadline=None)
@given(shape=SHAPES, scale=SCALES, seed=st.integers(0, 999))
def test_fp8_block128_is_a_projection_with_a_bounded_step(shape, scale, seed):
    w = _w(shape, scale, seed)
    q, s = C.fp8_quant_block128(w)
    d = C.fp8_dequant_block128(q, s)
    q2, s2 = C.fp8_quant_block128(d)
    assert torch.equal(C.fp8_dequant_block128(q2, s2), d)
    # E4M3 keeps 3 mantissa bits: half a step is 2^-4 of the value, plus the grid's floor at the block's scale
    amax = w.abs().max().item()
    assert ((d - w).abs() <= w.abs() * 2.0 ** -4 + amax * 2.0 ** -9 + 1e-12).all()
    qr, sr = C.fp8_quant_rows(w)
    dr = C.fp8_dequant_rows(qr, sr)
    assert torch.equal(C.fp8_dequant_rows(*C.fp8_quant_rows(dr)), dr)


@settings(max_examples=40, deadline=None)
@given(shape=SHAPES, scale=SCALES, seed=st.integers(0, 999))
def test_fp4_codecs_are_projections(shape, scale, seed):
    w = _w(shape, scale, seed)
    p, e = C.mxfp4_quant(w)
    d = C.mxfp4_dequant(p, e)
    assert torch.equal(C.mxfp4_dequant(*C.mxfp4_quant(d)), d)
    # E2M1's coarsest step is 2 (between 4 and 6) on a grid whose top is 6: a quarter of the group's scale at worst
    assert ((d - w).abs().view(-1, 32).amax(1) <= w.abs().view(-1, 32).amax(1) * 0.34 + 1e-12).all()
    p, b, gscale = C.nvfp4_quant(w)
    d = C.nvfp4_dequant(p, b, gscale)
    assert torch.isfinite(d).all() and d.shape == w.shape
    assert ((d - w).abs().view(-1, 16).amax(1) <= w.abs().view(-1, 16).amax(1) * 0.34 + w.abs().max() * 2.0 ** -6).all()


@given(data=st.lists(st.integers(0, 15), min_size=2, max_size=64).filter(lambda v: len(v) % 2 == 0))
def test_nibble_packing_is_lossless(data):
    codes = torch.tensor(data, dtype=torch.uint8).view(1, -1)
    assert torch.equal(C.unpack_nibbles(C.pack_nibbles(codes)), codes)


@settings(max_examples=20, deadline=None)
@given(rows=st.integers(1, 5), seed=st.integers(0, 99))
def test_hadamard128_is_an_involution_that_keeps_lengths(rows, seed):
    x = torch.randn(rows, 128, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)
    y = C.hadamard128(x)
    assert torch.allclose(C.hadamard128(y), x, atol=1e-9) and torch.allclose(y.norm(dim=1), x.norm(dim=1), atol=1e-9)
