import numpy as np
import torch

from cuteafd_b200.loader.mapped_table import MappedTable


def test_mapped_table_gather_prefetch_and_stats(tmp_path):
    rows, width = 5000, 48
    data = np.random.default_rng(0).standard_normal((rows, width)).astype(np.float16)
    path = tmp_path / "table.bin"
    with open(path, "wb") as f:
        f.write(b"\0" * 64)                       # a header before the table, like a tensor inside a checkpoint file
        f.write(data.tobytes())
    t = MappedTable(str(path), rows, width, np.float16, offset=64, workers=3, chunk_rows=100, cache_rows=1000)
    ids = np.random.default_rng(1).integers(0, rows, 777)
    out = t.gather(ids)
    assert torch.equal(out, torch.from_numpy(data[ids]))
    nxt = np.random.default_rng(2).integers(0, rows, 300)
    t.prefetch(nxt)
    out2 = t.gather(nxt)
    assert torch.equal(out2, torch.from_numpy(data[nxt]))
    assert t.stats.prefetch_hits == 300 and t.stats.gathers == 2 and t.stats.rows == 1077
    t.prefetch(np.arange(2000))                   # more than the cache holds: oldest rows fall out, reads stay right
    out3 = t.gather(np.arange(0, 2000, 7))
    assert torch.equal(out3, torch.from_numpy(data[np.arange(0, 2000, 7)]))
    t.close()
