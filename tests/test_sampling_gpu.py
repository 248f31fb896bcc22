"""The device sampler against the plain restatement of the reference's sampler."""
import pytest
import torch

import brolm_b200 as bb
from brolm_b200.sampling import uniform24
from tests.plain import sampling_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rows(n, vocab, seed, spread=4.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, vocab, generator=g) * spread


def test_greedy_picks_the_first_maximum():
    x = rows(6, 1001, 0)
    x[1, 17] = x[1, 900] = 99.0          # a tie: the lower id wins
    x[2, 0] = 50.0
    x[3, 1000] = 50.0
    for params in (bb.SamplingParams(temperature=0.0), bb.SamplingParams(temperature=-1.0),
                   bb.SamplingParams(temperature=0.7, top_k=1)):
        got = bb.Sampler(params)(x.to(DEV), torch.zeros(6, dtype=torch.int32, device=DEV), 0).tolist()
        assert got == [plain.greedy(r) for r in x] and got[1] == 17 and got[2] == 0 and got[3] == 1000


@pytest.mark.parametrize("n,vocab", [(1, 256000), (8, 256000), (3, 40004), (64, 65536), (200, 131072)])
def test_greedy_over_a_large_vocabulary(n, vocab):
    """Few rows of many values: several blocks fold a row and the last one to arrive writes the id.  Ties
    across blocks go to the lower id, negative maxima, infinities and NaN behave as in one block, and a
    second call finds the keys and counters at rest."""
    x = rows(n, vocab, n + vocab)
    x[0, vocab - 1] = x[0, 5] = 77.0                  # a tie between the first and the last block
    if n > 1:
        x[1] = -x[1].abs() - 1.0                      # all negative
        x[1, vocab // 2 + 3] = -0.5
    if n > 2:
        x[2, 11] = float("nan")
        x[2, vocab // 3] = float("inf")
        x[2, vocab - 2] = float("inf")
    sampler = bb.Sampler(bb.SamplingParams(temperature=0.0))
    streams = torch.zeros(n, dtype=torch.int32, device=DEV)
    want = [plain.greedy(torch.nan_to_num(r, nan=float("-inf"))) for r in x]      # a NaN is never greater: passed over
    assert want[0] == 5 and (n <= 2 or want[2] == vocab // 3)
    for _ in range(2):
        assert sampler(x.to(DEV), streams, 0).tolist() == want
    empty = torch.full((2, vocab), float("-inf"))
    assert sampler(empty.to(DEV), streams[:2], 0).tolist() == [0, 0]
    assert sampler(x.to(DEV), streams, 0).tolist() == want


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.8, 0, 1.0), (0.8, 5, 1.0), (1.3, 0, 0.7),
                                                     (0.5, 40, 0.9), (2.0, 3, 0.1), (1.0, 0, 0.0)])
@pytest.mark.parametrize("vocab", [500, 2048, 25601])
def test_draws_match_the_oracle(temperature, top_k, top_p, vocab):
    n, seed = 24, 7
    x = rows(n, vocab, vocab + top_k)
    streams = torch.arange(n, dtype=torch.int32) * 3 + 1
    sampler = bb.Sampler(bb.SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed))
    for counter in (0, 5):
        got = sampler(x.to(DEV), streams.to(DEV), counter).tolist()
        for r in range(n):
            u = uniform24(seed, int(streams[r]), counter)
            want = plain.sample(x[r], temperature, top_k, top_p, u)
            if got[r] != want:
                # only a draw that lands on the edge between two tokens may differ, and then by rounding alone
                probs, mask = plain.kept_set(x[r], temperature, top_k, top_p)
                assert bool(mask[got[r]]), "a token outside the kept set was drawn"
                kept = torch.where(mask, probs, torch.zeros_like(probs))
                acc = torch.cumsum(kept, 0) / kept.sum()
                lo = float(acc[got[r]] - kept[got[r]] / kept.sum())
                assert min(abs(u - lo), abs(u - float(acc[got[r]]))) < 1e-5, (r, got[r], want, u)


def test_equal_seeds_equal_draws_and_streams_differ():
    x = rows(8, 3000, 3).to(DEV)
    s = bb.Sampler(bb.SamplingParams(temperature=1.0, seed=11))
    streams = torch.arange(8, dtype=torch.int32, device=DEV)
    a, b = s(x, streams, 4).tolist(), s(x, streams, 4).tolist()
    assert a == b
    same_row = x[:1].repeat(8, 1).contiguous()
    draws = s(same_row, streams, 4).tolist()
    assert len(set(draws)) > 1                     # one distribution, eight streams: not all the same token


def test_frequencies_follow_the_distribution():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, -30.0]).repeat(1, 1)
    probs = torch.softmax(logits[0].double() / 0.9, 0)
    n = 4000
    x = logits.repeat(n, 1).contiguous().to(DEV)
    got = bb.Sampler(bb.SamplingParams(temperature=0.9, seed=5))(x, torch.arange(n, dtype=torch.int32, device=DEV), 1)
    freq = torch.bincount(got.cpu().long(), minlength=5).double() / n
    assert float((freq - probs).abs().max()) < 0.03
