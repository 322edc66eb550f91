"""Seeded generators: the same seed gives the same stream, different seeds differ
(mirrors legacy/examples/tensor/demo_seeds_and_determinism.mojo and demo_random.mojo)."""
import momijo.tensor as mt


def main():
    a, b, c = mt.rand([4], seed=7), mt.rand([4], seed=7), mt.rand([4], seed=8)
    ints = mt.randint([6], 0, 10, seed=3)
    perm = mt.creation.randperm_u16(5, 3)
    rng = mt.creation.RNG64(123)
    draws = [rng.next_i32(0, 6) for _ in range(5)]
    x = mt.zeros([2, 3])
    x.uniform_seeded(0.0, 1.0, 11)
    print(a.tolist(), ints.tolist(), perm.tolist(), draws, x.tolist())
    assert a.tolist() == b.tolist() != c.tolist() and sorted(perm.tolist()) == [0, 1, 2, 3, 4] and all(0 <= d < 6 for d in draws)
    return a


if __name__ == "__main__":
    main()
