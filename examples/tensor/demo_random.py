"""Seeded generators: same seed same numbers, different seeds differ, ranges respected
(legacy/examples/tensor/demo_random.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = mt.rand([4, 5], seed=123)
    b = mt.rand([4, 5], seed=123)
    c = mt.rand([4, 5], seed=124)
    g1, g2 = mt.init_rng(7), mt.init_rng(7)          # the reference's explicit generator object
    assert [g1.next_u64() for _ in range(3)] == [g2.next_u64() for _ in range(3)]
    assert a.tolist() == b.tolist() and a.tolist() != c.tolist()
    assert 0.0 <= a.min().item() and a.max().item() < 1.0
    n = mt.randn([2000], seed=5)
    assert abs(n.mean().item()) < 0.15 and 0.8 < n.std().item() < 1.2
    r = mt.randint([1000], 3, 9, seed=11)
    assert 3 <= r.min().item() and r.max().item() < 9
    p = mt.randperm_int(10)
    assert sorted(p.tolist()) == list(range(10))
    print("random ok")
    return True


if __name__ == "__main__":
    main()
