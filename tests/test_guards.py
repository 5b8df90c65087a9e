"""Guard bands around the regions of the symmetric exchange buffer."""
import torch

from cuteafd_b200.parallel.afd import GUARD, GUARD_BYTE, SymLayout, SymmetricHeap
from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry


def _heap(nbytes):
    h = object.__new__(SymmetricHeap)          # the band logic without a process group
    h.buf = torch.zeros(nbytes, dtype=torch.uint8)
    h.bands = []
    return h


def test_bands_sit_between_the_regions():
    geo = ExchangeGeometry(512, 256, 16, 4, max_tokens=300, n_expert_ranks=2, wave_tokens=128)
    lay = SymLayout.build(geo, num_layers=3, n_sources=2)
    bands = lay.guards(geo, 2)
    rg, n = geo.region(), geo.regions * 2
    assert len(bands) == 2 * n + 3
    payload = []
    for r in range(n):
        payload.append((lay.slab + r * lay.slab_stride(geo), rg.max_rows * geo.hidden * 2))
        payload.append((lay.meta + r * lay.meta_stride(geo), rg.meta_ints * 4))
    payload += [(lay.dflags, 3 * n * 4), (lay.combine, geo.max_tokens * geo.top_k * geo.hidden * 2), (lay.cflags, 3 * geo.regions * 8 * 4)]
    spans = sorted([(o, o + b, "data") for o, b in payload] + [(o, o + GUARD, name) for name, o in bands])
    for (a0, a1, _), (b0, b1, _) in zip(spans, spans[1:]):
        assert a1 <= b0, (a0, a1, b0, b1)                           # nothing overlaps
    assert spans[-1][1] == lay.total and spans[-1][2] == "completion flags"
    # every data region is followed by a band before the next data region starts
    kinds = [k for _, _, k in spans]
    assert all(not (a == "data" and b == "data") for a, b in zip(kinds, kinds[1:]))


def test_damage_is_named():
    geo = ExchangeGeometry(256, 128, 8, 2, max_tokens=64, n_expert_ranks=1)
    lay = SymLayout.build(geo, num_layers=2)
    h = _heap(lay.total)
    h.arm(lay.guards(geo))
    assert h.damaged() == [] and int(h.buf[lay.total - 1]) == GUARD_BYTE
    rg = geo.region()
    h.buf[lay.slab + rg.max_rows * geo.hidden * 2 - 1] = 7          # last payload byte of the slab: fine
    assert h.damaged() == []
    h.buf[lay.slab + lay.slab_stride(geo) - GUARD + 5] = 7          # one byte past the slab's rows
    h.buf[lay.total - 1] = 0
    assert h.damaged() == ["slab[0]", "completion flags"]
