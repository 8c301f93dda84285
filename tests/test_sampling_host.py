"""The host-side sampling rule against the plain sampler (CPU)."""
import numpy as np
import pytest
import torch

import plain_lfm2 as P
from gesso_b200.errors import ErrorCode, GessoError
from gesso_b200.sampling import SamplingParams, SplitMix64, greedy_host, sample_host


def test_splitmix_matches_plain():
    a, b = SplitMix64(123), P.PlainSampler(1.0, 1.0, 123)
    assert [a.unit() for _ in range(10)] == [b.unit() for _ in range(10)]
    assert all(0.0 <= SplitMix64(s).unit() < 1.0 for s in range(100))


@pytest.mark.parametrize("kind", ["random", "flat", "peaked", "tied", "underflow"])
@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.3])
def test_host_rule_equals_plain_full_sort(kind, top_p):
    """Flat, peaked, tied and underflowing rows (test/test_sampling.jl:107-125)."""
    g = torch.Generator().manual_seed(11)
    V = 700
    row = {"random": 2 * torch.randn(V, generator=g), "flat": torch.zeros(V),
           "peaked": torch.cat([torch.tensor([50.0]), torch.randn(V - 1, generator=g)]),
           "tied": torch.round(torch.randn(V, generator=g)),
           "underflow": torch.cat([torch.tensor([0.0, -1.0]), torch.full((V - 2,), -2000.0)])}[kind].numpy().astype(np.float32)
    for seed in range(8):
        p = SamplingParams(0.9, top_p, seed)
        rng, plain = SplitMix64(seed), P.PlainSampler(0.9, top_p, seed)
        for _ in range(5):
            assert sample_host(row, p, rng) == plain.sample(row.tolist())


def test_greedy_ties_and_nonfinite():
    assert greedy_host(np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32)) == 1
    for bad in (np.nan, np.inf, -np.inf):
        with pytest.raises(GessoError) as e:
            greedy_host(np.array([0.0, bad], dtype=np.float32))
        assert e.value.code == ErrorCode.NUMERICAL_INSTABILITY
        with pytest.raises(GessoError):
            sample_host(np.array([0.0, bad], dtype=np.float32), SamplingParams(1.0), SplitMix64(0))
    assert sample_host(np.array([0.0, 5.0, 1.0], dtype=np.float32), SamplingParams(0.0), None) == 1
