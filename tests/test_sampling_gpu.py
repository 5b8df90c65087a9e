"""GPU target sampler and accept-prefix scan against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sample_rows_match_oracle():
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.sampling import SamplingParams, select_rows
    dev = torch.device("cuda", 0)
    V = 5003
    g = torch.Generator().manual_seed(0)
    cases = [SamplingParams(), SamplingParams(temperature=0.7, seed=1), SamplingParams(temperature=1.0, top_k=5, seed=2),
             SamplingParams(temperature=1.3, top_p=0.9, seed=3), SamplingParams(temperature=0.9, min_p=0.05, seed=4),
             SamplingParams(temperature=1.0, top_k=50, top_p=0.8, min_p=0.01, seed=5), SamplingParams(temperature=2.0, top_k=1, seed=6),
             SamplingParams(temperature=0.3, top_p=0.5, seed=7), SamplingParams(temperature=1.0, top_k=V + 10, seed=8)]
    params, positions = [], []
    for rep in range(6):
        for c in cases:
            params.append(SamplingParams(c.temperature, c.top_p, c.top_k, c.min_p, c.seed + 100 * rep))
            positions.append(17 + 1000 * rep + len(params))
    n = len(params)
    logits = torch.randn(n, V, generator=g) * 3.0
    logits[3, 100:110] = logits[3].max() + 1.0            # a block of exact ties at the top
    logits[5, ::7] = 2.5                                  # many ties in the middle
    masks = [None] * n
    words = (V + 31) // 32
    mask_bits = torch.zeros(n, words, dtype=torch.int32)
    mask_word0 = [None] * n
    for i in range(0, n, 4):
        m = torch.rand(V, generator=g) < 0.3
        m[int(torch.randint(0, V, (1,), generator=g))] = True
        masks[i] = m
        padded = torch.zeros(words * 32, dtype=torch.bool); padded[:V] = m
        w = (padded.view(words, 32).long() << torch.arange(32)).sum(1)
        mask_bits[i] = torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)
        mask_word0[i] = i * words
    want, want_status = select_rows(logits, params, positions, masks)
    rows = K.pack_sample_rows(params, positions, mask_word0=mask_word0).to(dev)
    tok = torch.full((n,), -7, dtype=torch.int32, device=dev)
    st = torch.full((n,), -7, dtype=torch.int32, device=dev)
    for _ in range(2):
        K.sample_rows(logits.to(dev), rows, tok, st, mask_bits.to(dev))
    torch.cuda.synchronize()
    assert st.tolist() == want_status
    got = tok.tolist()
    bad = [i for i in range(n) if got[i] != want[i]]
    assert not bad, [(i, got[i], want[i], params[i]) for i in bad[:5]]


def test_sample_row_errors_and_accept_prefix():
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.sampling import STATUS_EMPTY_MASK, STATUS_NONFINITE, SamplingParams, accept_prefix
    dev = torch.device("cuda", 0)
    V = 300
    logits = torch.randn(3, V)
    logits[1, 5] = float("nan")
    mask_bits = torch.zeros(3, (V + 31) // 32, dtype=torch.int32)
    params = [SamplingParams(temperature=1.0)] * 3
    rows = K.pack_sample_rows(params, [0, 1, 2], mask_word0=[None, None, 2 * mask_bits.shape[1]]).to(dev)
    tok = torch.zeros(3, dtype=torch.int32, device=dev); st = torch.zeros(3, dtype=torch.int32, device=dev)
    K.sample_rows(logits.to(dev), rows, tok, st, mask_bits.to(dev))
    assert st.tolist() == [0, STATUS_NONFINITE, STATUS_EMPTY_MASK] and tok.tolist()[1:] == [-1, -1]
    # accept-prefix: three sequences with 4, 1 and 3 rows
    selected = [5, 6, 7, 8, 9, 1, 2, 3]
    draft = [5, 6, 0, 0, 0, 1, 2, 0]
    row_start = [0, 4, 5, 8]
    i32 = dict(dtype=torch.int32, device=dev)
    acc = torch.zeros(3, **i32); bonus = torch.zeros(3, **i32)
    K.accept_prefix(torch.tensor(selected, **i32), torch.tensor(draft, **i32), torch.tensor(row_start, **i32), acc, bonus)
    want = [accept_prefix(selected[a:b], draft[a:b - 1]) for a, b in zip(row_start[:-1], row_start[1:])]
    assert list(zip(acc.tolist(), bonus.tolist())) == want
