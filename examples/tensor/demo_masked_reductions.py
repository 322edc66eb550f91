"""Reductions over the elements selected by a mask, and NaN-aware reductions
(legacy/examples/tensor/demo_masked_reductions.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = np.array([[1.0, -2.0, 3.0], [4.0, np.nan, -6.0]])
    t = mt.Tensor(a.tolist())
    pos = (t > 0).bool()
    assert t[pos].sum().item() == 8.0
    assert mt.where(pos, t, mt.zeros_like(t)).sum(0).tolist() == [5.0, 0.0, 3.0]
    assert mt.nanops.nansum(t).item() == 0.0
    assert abs(mt.nanops.nanmean(t).item() - 0.0) < 1e-12
    filled = mt.nanops.nan_to_num(t, 0.0)
    assert filled.tolist() == [[1.0, -2.0, 3.0], [4.0, 0.0, -6.0]]
    cnt = pos.sum().item()
    print("masked sum 8.0 over", cnt, "elements")
    return cnt


if __name__ == "__main__":
    main()
