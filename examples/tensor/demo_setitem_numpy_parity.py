"""Assignment through selectors on 1-D .. 4-D tensors, checked element by element against NumPy
(legacy/examples/tensor/demo_setitem_numpy_parity.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    checks = 0
    shapes = [(12,), (4, 5), (2, 3, 4), (2, 3, 4, 5)]
    for shp in shapes:
        a = np.arange(int(np.prod(shp)), dtype=np.float64).reshape(shp)
        t = mt.Tensor(a.tolist())
        nd = len(shp)
        cases = [(Ellipsis, -1.0), ((0,) + (slice(None),) * (nd - 1), 5.0)]
        if nd >= 2:
            cases += [((slice(None), slice(1, None, 2)), 9.0), ((slice(None, None, -1), 0), 2.5),
                      ((slice(0, 1), Ellipsis), -3.0), ((-1, -1), 11.0)]
        if nd >= 3:
            cases += [((slice(None), 1, slice(None, None, 2)), 4.0), ((0, Ellipsis, -1), 6.0),
                      ((slice(None), [0, 2]), 8.0)]
        if nd == 4:
            cases += [((1, slice(None), 2, slice(1, 4)), 1.5), ((slice(None), slice(None), slice(None), [0, 4]), 0.25)]
        for sel, val in cases:
            a[sel] = val
            t[sel] = val
            assert np.array_equal(np.asarray(t.tolist()), a), (shp, sel)
            checks += 1
        # tensor-valued right-hand sides broadcast like NumPy
        if nd >= 2:
            row = np.arange(shp[-1], dtype=np.float64)
            a[0] = row
            t[0] = mt.Tensor(row.tolist())
            assert np.array_equal(np.asarray(t.tolist()), a)
            checks += 1
    # boolean masks
    a = np.arange(20, dtype=np.float64).reshape(4, 5)
    t = mt.Tensor(a.tolist())
    a[a > 12] = 0
    t[(t > 12).bool()] = 0   # comparisons give 0/1 tensors (the reference's masks); .bool() selects by mask
    assert np.array_equal(np.asarray(t.tolist()), a)
    checks += 1
    # string selectors of the reference: S("1:3, :")
    b = np.arange(20, dtype=np.float64).reshape(4, 5)
    u = mt.Tensor(b.tolist())
    b[1:3, ::2] = -7
    u[mt.S("1:3, ::2")] = -7
    assert np.array_equal(np.asarray(u.tolist()), b)
    checks += 1
    print("setitem parity checks passed:", checks)
    return checks


if __name__ == "__main__":
    main()
