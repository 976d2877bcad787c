"""Every privacy sampler on its own (the layout of packages/opake-dpsgd/tests/sampling and packages/opake-dpftrl/tests/
sampling): statistical contract, determinism in the key, argument validation, resumption at every position."""
import numpy as np
import pytest

from opake_b200.base.exceptions import ConfigurationError
from opake_b200.base.serialization import from_state_dict, state_dict
from opake_b200.dpftrl.sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler, SequentialBatchSampler
from opake_b200.dpsgd.sampling import KOutOfTSampler, PoissonSampler
from opake_b200.engine.random import key

N = 600
DATA = list(range(N))

_MAKERS = {
    "poisson": lambda k: PoissonSampler(DATA, 0.05, n_steps=14, key=k),
    "poisson_truncated": lambda k: PoissonSampler(DATA, 0.2, n_steps=14, truncated_batch_size=50, key=k),
    "k_out_of_t_block": lambda k: KOutOfTSampler(DATA, k=2, t=14, allocation="block", key=k),
    "k_out_of_t_total": lambda k: KOutOfTSampler(DATA, k=3, t=14, allocation="total", key=k),
    "cyclic_poisson": lambda k: CyclicPoissonSampler(DATA, 0.3, bands=4, n_steps=14, key=k),
    "b_min_sep": lambda k: BMinSepSampler(DATA, 3, 0.2, 14, key=k),
    "balls_in_bins": lambda k: BallsInBinsSampler(DATA, 7, 14, key=k),
    "sequential": lambda k: SequentialBatchSampler(DATA, 50, 14),
}


@pytest.mark.parametrize("name", list(_MAKERS))
def test_same_key_same_stream_other_key_other_stream(name):
    a, b = list(_MAKERS[name](key(1))), list(_MAKERS[name](key(1)))
    assert a == b and len(a) == 14
    assert all(all(0 <= i < N for i in batch) for batch in a)
    assert all(len(set(batch)) == len(batch) for batch in a)                # no example twice in one batch
    if name != "sequential":
        assert list(_MAKERS[name](key(2))) != a


@pytest.mark.parametrize("name", list(_MAKERS))
@pytest.mark.parametrize("cut", [0, 1, 5, 13])
def test_resume_at_any_position_reproduces_the_tail(name, cut):
    s = _MAKERS[name](key(3))
    it = iter(s)
    head = [next(it) for _ in range(cut)]
    sd = dict(state_dict(s))
    tail = list(it)
    fresh = from_state_dict(_MAKERS[name](key(99)), sd)           # the stream key travels in the state
    assert list(fresh) == tail and len(head) + len(tail) == 14


def test_poisson_inclusion_rate_and_truncation():
    q, steps = 0.05, 400
    counts = np.zeros(N)
    sizes = []
    for b in PoissonSampler(DATA, q, n_steps=steps, key=key(4)):
        counts[b] += 1
        sizes.append(len(b))
    assert abs(np.mean(sizes) - q * N) < 3 * np.sqrt(q * (1 - q) * N / steps) + 0.5
    assert abs(counts.mean() / steps - q) < 0.005 and counts.min() > 0
    # independent across steps: the variance of the batch size is binomial
    assert 0.7 < np.var(sizes) / (N * q * (1 - q)) < 1.3
    capped = [len(b) for b in PoissonSampler(DATA, 0.2, n_steps=100, truncated_batch_size=100, key=key(4))]
    assert max(capped) <= 100 and min(capped) > 60 and any(c == 100 for c in capped)


@pytest.mark.parametrize("allocation", ["block", "total"])
def test_k_out_of_t_every_example_exactly_k_times(allocation):
    k, t = 3, 12
    counts = np.zeros(N, int)
    batches = list(KOutOfTSampler(DATA, k=k, t=t, allocation=allocation, key=key(5)))
    assert len(batches) == t
    for b in batches:
        counts[b] += 1
    assert (counts == k).all()
    if allocation == "block":            # one participation per block of t / k steps
        block = t // k
        for j in range(k):
            c = np.zeros(N, int)
            for b in batches[j * block:(j + 1) * block]:
                c[b] += 1
            assert (c == 1).all()


def test_cyclic_poisson_respects_the_band_partition():
    bands, steps = 4, 16
    s = CyclicPoissonSampler(DATA, 0.5, bands=bands, n_steps=steps, key=key(6))
    batches = list(s)
    seen_in = [set() for _ in range(bands)]
    for t, b in enumerate(batches):
        seen_in[t % bands].update(b)
    for i in range(bands):
        for j in range(i + 1, bands):
            assert not (seen_in[i] & seen_in[j])           # an example only ever appears in its own residue class
    assert sum(len(x) for x in seen_in) > 0.9 * N          # q = 0.5 over 4 visits: 94 % expected coverage


def test_b_min_sep_never_reuses_an_example_within_the_separation():
    b = 3
    batches = list(BMinSepSampler(DATA, b, 0.3, 20, key=key(7)))
    last = {}
    for t, batch in enumerate(batches):
        for i in batch:
            assert i not in last or t - last[i] >= b, (i, t, last[i])
            last[i] = t
    assert len(last) > 0.8 * N


def test_balls_in_bins_is_a_fixed_partition_cycled():
    bins = list(BallsInBinsSampler(DATA, 5, 15, key=key(8)))
    assert bins[:5] == bins[5:10] == bins[10:]
    assert sorted(i for b in bins[:5] for i in b) == DATA
    sizes = [len(b) for b in bins[:5]]
    assert max(sizes) - min(sizes) < 60                    # multinomial allocation, not equal split


def test_sequential_batches_cover_the_data_in_order():
    batches = list(SequentialBatchSampler(DATA, 64, 12))
    flat = [i for b in batches for i in b]
    assert flat[:N] == DATA[: len(flat[:N])] and all(len(b) <= 64 for b in batches)


@pytest.mark.parametrize("bad", [lambda: PoissonSampler(DATA, 0.0, key=key(0)), lambda: PoissonSampler(DATA, 1.5, key=key(0)),
                                 lambda: PoissonSampler(DATA, 0.1, n_steps=0, key=key(0)),
                                 lambda: PoissonSampler(DATA, 0.1, truncated_batch_size=0, key=key(0)),
                                 lambda: KOutOfTSampler(DATA, k=5, t=3, allocation="total", key=key(0)),
                                 lambda: KOutOfTSampler(DATA, k=2, t=8, allocation="diagonal", key=key(0))])
def test_invalid_arguments_are_configuration_errors(bad):
    with pytest.raises((ConfigurationError, ValueError)):
        bad()


def test_state_of_another_dataset_is_refused():
    s = PoissonSampler(DATA, 0.1, n_steps=5, key=key(1))
    next(iter(s))
    with pytest.raises(ValueError):
        from_state_dict(PoissonSampler(DATA[:100], 0.1, n_steps=5, key=key(1)), dict(state_dict(s)))
