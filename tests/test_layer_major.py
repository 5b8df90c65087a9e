"""Layer-major oracle run: equal to the whole forward pass, resumable after an interruption between layers with the same
bytes at the end, and unwilling to continue a directory made for other tokens."""
import os

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.loader.load import load_params
from cuteafd_b200.loader.snapshot import write_random_snapshot
from cuteafd_b200.ref import layer_major as LM
from cuteafd_b200.ref.model import KvState, RefDecoder


@pytest.mark.parametrize("fmt", ["bf16", "fp8_block128"])
def test_layer_major_run_matches_the_whole_forward_and_resumes(fmt, tmp_path):
    cfg = tiny_moe().replace(num_layers=3)
    snap = write_random_snapshot(cfg, str(tmp_path / "snap"), fmt=fmt, seed=2, scope="linear" if fmt != "bf16" else "experts")
    toks = torch.randint(0, cfg.vocab_size, (2, 20), generator=torch.Generator().manual_seed(1))
    out = str(tmp_path / "run")

    class Stop(Exception):
        pass

    def die_after_first(i):
        if i == 0:
            raise Stop()
    with pytest.raises(Stop):
        LM.run(snap, toks, out, after_layer=die_after_first)
    assert os.path.exists(os.path.join(out, "layer00.bin")) and not os.path.exists(os.path.join(out, "layer01.bin"))
    seen = []
    LM.run(snap, toks, out, after_layer=seen.append)
    assert seen == [1, 2]                                      # layer 0 was not computed again
    got = LM.read(out)
    _, params = load_params(snap)
    ref = RefDecoder(cfg, params)
    with torch.no_grad():
        for w in range(2):
            want = ref.forward(toks[w], KvState(cfg))
            assert torch.allclose(got["logits"][w], want, atol=1e-4, rtol=1e-4)
    assert torch.equal(got["tokens"], toks) and len(got["layers"]) == 3 and got["layers"][0].shape == (2, 20, cfg.hidden)
    # a straight run in a fresh directory writes the same bytes
    out2 = str(tmp_path / "run2")
    LM.run(snap, toks, out2)
    for name in ("layer00.bin", "layer02.bin", "logits.bin", "tokens.bin"):
        assert open(os.path.join(out, name), "rb").read() == open(os.path.join(out2, name), "rb").read(), name
    with pytest.raises(ValueError):
        LM.run(snap, toks + 1, out)
