import numpy as np

from triebwerk_b200.partition import contiguous_partition, lpt_partition, partition_loads


def test_contiguous_partition_covers_everything_once():
    for n, w in ((64, 8), (10, 4), (3, 8), (256, 2)):
        parts = contiguous_partition(n, w)
        flat = [i for p in parts for i in p]
        assert flat == list(range(n))
        sizes = [len(p) for p in parts]
        assert max(sizes) - min(sizes) <= 1


def test_lpt_balances_ragged_lengths():
    lengths = np.random.default_rng(0).integers(128, 16385, 1024)
    for w in (2, 4, 8):
        parts = lpt_partition(lengths, w)
        flat = sorted(i for p in parts for i in p)
        assert flat == list(range(1024))
        loads = partition_loads(lengths, parts)
        assert max(loads) - min(loads) <= lengths.max()
        assert max(loads) <= 1.01 * (sum(loads) / w)
        assert all(p == sorted(p) for p in parts)
    assert lpt_partition(lengths, 8) == lpt_partition(lengths, 8)  # deterministic


def test_lpt_with_more_ranks_than_sequences():
    parts = lpt_partition([5, 9], 4)
    assert sorted(len(p) for p in parts) == [0, 0, 1, 1]
