"""Second parity sweep: negative steps, ellipsis, new axes, integer-array and boolean indexing, take / gather /
where / nonzero against NumPy (legacy/examples/tensor/demo_indexing_numpy_parity2.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    checks = 0
    a = np.arange(3 * 4 * 5, dtype=np.float64).reshape(3, 4, 5)
    t = mt.Tensor(a.tolist())
    sels = [
        (slice(None, None, -1),), (slice(None), slice(None, None, -2)), (Ellipsis, slice(4, 0, -1)),
        (None, 1, Ellipsis), (slice(1, 3), None, 2), (-1, -2, -3), ([2, 0],), (slice(None), [3, 1, 1]),
        (slice(None), slice(None), [0, 0, 4]), (1, slice(-3, None)), (Ellipsis, None),
    ]
    for sel in sels:
        got, ref = t[sel], a[sel]
        assert tuple(got.shape) == ref.shape, sel
        assert np.array_equal(np.asarray(got.tolist()).reshape(ref.shape), ref), sel
        checks += 1
    m = a % 3 == 0
    assert np.array_equal(np.asarray(t[(t % 3 == 0).bool()].tolist()), a[m])
    checks += 1
    idx = np.array([[0, 2], [1, 1], [3, 0]])
    ti = mt.Tensor(idx.tolist()).long()
    assert np.array_equal(np.asarray(mt.take(t, mt.Tensor([1, 7, 59]).long()).tolist()), np.take(a, [1, 7, 59]))
    g = mt.gather(t[0], 0, ti[:, :1].expand(3, 5))
    assert np.array_equal(np.asarray(g.tolist()), np.take_along_axis(a[0], idx[:, :1].repeat(5, 1), 0))
    checks += 2
    w = mt.where((t > 30).bool(), t, -t)
    assert np.array_equal(np.asarray(w.tolist()), np.where(a > 30, a, -a))
    nz = mt.nonzero((t[0] > 12).bool())
    assert np.array_equal(np.asarray(nz.tolist()), np.argwhere(a[0] > 12))
    checks += 2
    print("indexing parity (2) checks passed:", checks)
    return checks


if __name__ == "__main__":
    main()
