"""Image preprocessing on generated sizes: the resized grid is whole merged cells inside the pixel budget with the aspect
kept as closely as the cell size allows, every patch row is where ``patch_positions`` says, and identical pixels give
identical rows whatever surrounds the call."""
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.media.image import MediaError, patch_positions, preprocess_image, smart_resize


@settings(max_examples=300)
@given(h=st.integers(1, 5000), w=st.integers(1, 5000), factor=st.sampled_from([28, 32]),
       lo=st.sampled_from([56 * 56, 4 * 28 * 28]), hi=st.sampled_from([256 * 28 * 28, 1280 * 28 * 28]))
def test_resize_targets_are_whole_cells_inside_the_budget(h, w, factor, lo, hi):
    if max(h, w) / min(h, w) > 200:
        try:
            smart_resize(h, w, factor, lo, hi)
            raise AssertionError("accepted a 200:1 strip")
        except MediaError:
            return
    nh, nw = smart_resize(h, w, factor, lo, hi)
    assert nh % factor == 0 and nw % factor == 0 and nh >= factor and nw >= factor
    assert nh * nw <= hi or (nh == factor or nw == factor)             # a strip one cell wide may exceed nothing else
    if h * w >= lo and min(h, w) >= factor:
        assert nh * nw >= min(lo, (h // factor) * (w // factor) * factor * factor) * 0.5
    # the aspect moves by at most one cell in each direction
    if min(nh, nw) > factor:
        assert abs(nh / nw - h / w) <= (h / w) * (factor / min(nh, nw)) * 2 + 1e-9


@settings(max_examples=25, deadline=None)
@given(h=st.integers(20, 200), w=st.integers(20, 200), seed=st.integers(0, 99))
def test_patch_rows_sit_where_patch_positions_says(h, w, seed):
    px = torch.randint(0, 256, (h, w, 3), generator=torch.Generator().manual_seed(seed), dtype=torch.uint8)
    rows, (gh, gw) = preprocess_image(px, patch=14, merge=2, min_pixels=4 * 28 * 28, max_pixels=64 * 28 * 28)
    assert rows.shape == (gh * gw, 3 * 14 * 14) and gh % 2 == 0 and gw % 2 == 0 and torch.isfinite(rows).all()
    pos = patch_positions(gh, gw, 2)
    assert sorted(map(tuple, pos.tolist())) == [(r, c) for r in range(gh) for c in range(gw)]       # every patch exactly once
    for cell in range(0, gh * gw, 4):                                                               # a merged cell is 2 x 2 neighbours
        rr, cc = pos[cell:cell + 4, 0], pos[cell:cell + 4, 1]
        assert int(rr.max() - rr.min()) == 1 and int(cc.max() - cc.min()) == 1
    again, _ = preprocess_image(px.clone(), patch=14, merge=2, min_pixels=4 * 28 * 28, max_pixels=64 * 28 * 28)
    assert torch.equal(rows, again)
