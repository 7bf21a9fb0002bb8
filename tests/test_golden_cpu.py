"""The committed golden fixture still matches what the oracle computes from
the same seeds (guards the oracle and the input generator against drift)."""
import numpy as np

from tests.golden import make_golden as mg

GOLD = np.load(mg.Path(mg.__file__).with_name("matmul_golden.npz"))


def test_fixture_matches_oracle_bit_for_bit():
    for name, kind, m, k, n, batch, lsk, rsk, seed in mg.CASES:
        l, r, ls, rs = mg.make_inputs(kind, m, k, n, batch, lsk, rsk, seed)
        assert bytes(GOLD[name + "/sha"]).decode() == mg.digest(l, r), f"{name}: input generator drifted"
        y = np.ascontiguousarray(mg.expected(kind, l, r, m, k, n, batch, ls, rs), np.float32).reshape(-1)
        assert np.array_equal(y.view(np.uint32), GOLD[name + "/y"].view(np.uint32)), name
