"""Integer, slice and ellipsis selectors, item access, row / column helpers
(legacy/examples/tensor/demo_indexing.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = np.arange(24).reshape(2, 3, 4)
    t = mt.Tensor(a.tolist())
    assert t[1, 2, 3].item() == 23 and t[0].tolist() == a[0].tolist()
    assert t[:, 1].tolist() == a[:, 1].tolist() and t[..., 0].tolist() == a[..., 0].tolist()
    assert t[1, 1:, ::2].tolist() == a[1, 1:, ::2].tolist()
    m = mt.Tensor(a[0].tolist())
    assert mt.row(m, 1).tolist() == a[0][1].tolist() and mt.col(m, 2).tolist() == a[0][:, 2].tolist()
    assert mt.head(m, 2).tolist() == a[0][:2].tolist() and mt.tail(m, 1).tolist() == a[0][-1:].tolist()
    assert mt.slice1d(mt.Tensor(list(range(10))), 2, 8, 2).tolist() == [2, 4, 6]
    print("indexing ok")
    return True


if __name__ == "__main__":
    main()
