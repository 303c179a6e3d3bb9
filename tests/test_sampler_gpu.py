"""GPU sampler against the host oracle: every filter combination, masks, ties, error statuses."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle(logits, mask, p):
    from ds41rt_b200.runtime import core
    u = core.sample_uniform(p.seed, p.position)
    try:
        return core.sample_token(logits, mask, p.temperature, p.top_k, p.top_p, p.min_p, u), 0
    except core.SamplingError as e:
        return -1, str(e)


@pytest.mark.parametrize("vocab", [1000, 4096, 129280])
def test_sampler_matches_host_oracle(vocab):
    from ds41rt_b200.ops.sampling import RowParams, pack_params, sample_rows
    rng = np.random.default_rng(vocab)
    combos = [dict(temperature=0.0), dict(temperature=1.0), dict(temperature=0.7, top_k=40),
              dict(temperature=1.3, top_p=0.9), dict(temperature=0.8, top_k=50, top_p=0.95),
              dict(temperature=1.0, min_p=0.05), dict(temperature=0.9, min_p=0.02, top_k=20, top_p=0.8),
              dict(temperature=2.0, top_k=1), dict(temperature=1.0, top_k=5000), dict(temperature=1.0, top_p=0.3)]
    rows = 4 * len(combos)
    logits = rng.normal(0, 3, size=(rows, vocab)).astype(np.float32)
    logits[3] = np.round(logits[3])              # heavy ties
    logits[5] = np.round(logits[5] * 2) / 2
    logits[7, ::3] = -np.inf
    words = (vocab + 31) // 32
    masks = rng.integers(0, 2 ** 32, size=(3, words), dtype=np.uint64).astype(np.uint32)
    masks[1] &= rng.integers(0, 2 ** 32, size=words, dtype=np.uint64).astype(np.uint32)
    masks[2] = 0
    masks[2, 5] = 0b1011                         # three candidates only
    params = []
    for r in range(rows):
        c = combos[r % len(combos)]
        params.append(RowParams(seed=1234 + r, position=r * 7, mask_row=[-1, 0, 1, 2][r // len(combos)], **c))
    dev = torch.device("cuda")
    tok, st = sample_rows(torch.from_numpy(logits).to(dev), pack_params(params, dev),
                          torch.from_numpy(masks.view(np.int32)).to(dev))
    tok2, _ = sample_rows(torch.from_numpy(logits).to(dev), pack_params(params, dev),
                          torch.from_numpy(masks.view(np.int32)).to(dev))
    torch.cuda.synchronize()
    assert torch.equal(tok, tok2)
    tok, st = tok.cpu().numpy(), st.cpu().numpy()
    mismatches = 0
    for r, p in enumerate(params):
        m = masks[p.mask_row] if p.mask_row >= 0 else None
        want, err = _oracle(logits[r], m, p)
        assert (st[r] == 0) == (err == 0), (r, st[r], err)
        if err == 0 and tok[r] != want:
            mismatches += 1                      # only a draw that lands on a cumulative boundary may differ
    assert mismatches <= 1, mismatches


def test_sampler_statuses():
    from ds41rt_b200.ops.sampling import RowParams, pack_params, sample_rows
    dev = torch.device("cuda")
    vocab = 512
    logits = torch.randn(5, vocab, device=dev)
    logits[1, 7] = float("nan")
    logits[2, 9] = float("inf")
    masks = torch.zeros(1, vocab // 32, dtype=torch.int32, device=dev)
    params = [RowParams(temperature=-1.0), RowParams(temperature=0.0), RowParams(temperature=1.0),
              RowParams(temperature=1.0, mask_row=0), RowParams(temperature=1.0, top_p=0.0)]
    tok, st = sample_rows(logits, pack_params(params, dev), masks)
    assert st.tolist() == [3, 2, 2, 1, 6]


def test_sampler_adversarial_rows_match_host_oracle():
    """Rows built to sit on the sampler's decision boundaries (ideas from the reference's selftest,
    native/tests/v41_sampling_selftest.cu): ties straddling the top-k cut, k beyond the in-register selection width,
    all-equal rows, one dominant token, scaled values that fall into the subnormal range, huge negative logits, a
    single allowed token, an empty mask, min_p = 1, top_p at a cumulative boundary, near-greedy temperatures and a
    vocabulary that is not a multiple of 32.  Every row is drawn with four seeds and must equal the host oracle's
    token (or its error)."""
    from ds41rt_b200.ops.sampling import RowParams, pack_params, sample_rows
    rng = np.random.default_rng(7)
    vocab = 5003                                     # not a multiple of 32: the last mask word is partial
    words = (vocab + 31) // 32
    base = rng.normal(0, 2, size=vocab).astype(np.float32)
    rows, params = [], []

    def add(logit_row, mask_row=-1, **kw):
        for s in range(4):
            rows.append(np.asarray(logit_row, dtype=np.float32))
            params.append(RowParams(seed=99 + 17 * s + len(rows), position=3 * len(rows) + s, mask_row=mask_row, **kw))

    tie = base.copy()
    tie[100:160] = 5.0                               # 60 equal values on top: every cut below 60 splits the tie
    for k in (1, 7, 40, 59, 60, 61):
        add(tie, temperature=1.0, top_k=k)
    add(tie, temperature=0.7, top_k=50, top_p=0.5)
    for k in (256, 257, 300, 1000, vocab, vocab + 10):       # selection width boundary and no-op widths
        add(base, temperature=1.0, top_k=k)
    add(np.zeros(vocab), temperature=1.0)                     # all equal
    add(np.zeros(vocab), temperature=1.0, top_k=33, top_p=0.9)
    peak = base.copy()
    peak[4321] = 80.0                                        # one dominant token: everything else underflows
    add(peak, temperature=1.0)
    add(peak, temperature=1.0, top_p=0.999)
    add(base * 1e-30, temperature=2.0)                       # scaled differences are subnormal
    add(base * 1e-38, temperature=1.0, top_k=10)
    neg = base.copy()
    neg[::2] = -1e30                                         # finite but astronomically unlikely
    add(neg, temperature=1.0, top_p=0.95)
    add(base, temperature=1.0, min_p=1.0)                    # only the maxima survive
    add(tie, temperature=1.0, min_p=1.0)
    two = np.full(vocab, -50.0, dtype=np.float32)
    two[10], two[20] = 0.0, 0.0                              # two tokens at 0.5 each: top_p = 0.5 sits on the boundary
    add(two, temperature=1.0, top_p=0.5)
    add(two, temperature=1.0, top_p=0.5000001)
    for t in (1e-6, 9e-6, 1.1e-5, 1e-4, 1e-3):               # around the greedy threshold
        add(base, temperature=t)
    masks = np.zeros((3, words), dtype=np.uint32)
    masks[0, words - 1] = 1 << ((vocab - 1) % 32)            # only the last token of the vocabulary
    masks[1] = 0                                             # nothing allowed
    masks[2] = rng.integers(0, 2 ** 32, size=words, dtype=np.uint64).astype(np.uint32)
    masks[2, words - 1] &= (1 << (vocab % 32)) - 1
    add(base, mask_row=0, temperature=1.0, top_k=5)
    add(base, mask_row=0, temperature=0.0)
    add(base, mask_row=1, temperature=1.0)
    add(tie, mask_row=2, temperature=1.0, top_k=30)
    add(tie, mask_row=2, temperature=0.0)                    # masked greedy with ties: lowest allowed id
    logits = np.stack(rows)
    dev = torch.device("cuda")
    tok, st = sample_rows(torch.from_numpy(logits).to(dev), pack_params(params, dev),
                          torch.from_numpy(masks.view(np.int32)).to(dev))
    torch.cuda.synchronize()
    tok, st = tok.cpu().numpy(), st.cpu().numpy()
    bad = []
    for r, p in enumerate(params):
        m = masks[p.mask_row] if p.mask_row >= 0 else None
        want, err = _oracle(logits[r], m, p)
        if (st[r] == 0) != (err == 0) or (err == 0 and tok[r] != want):
            bad.append((r, int(st[r]), int(tok[r]), want, err))
    assert not bad, bad[:8]
