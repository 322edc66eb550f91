"""In-place updates change the storage that views share; out-of-place ops do not
(legacy/examples/tensor/demo_inplace_notes.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    t = mt.zeros([2, 3])
    v = t[0]
    v += 1.0                      # in place through a view
    assert t.tolist() == [[1.0, 1.0, 1.0], [0.0, 0.0, 0.0]]
    u = t + 5.0                   # new storage
    u[0, 0] = -1.0
    assert t[0, 0].item() == 1.0
    t.mul_(2.0)
    t[1].fill_(7.0)
    assert t.tolist() == [[2.0, 2.0, 2.0], [7.0, 7.0, 7.0]]
    c = t.clone()
    c.zero_()
    assert t.sum().item() == 27.0
    print("in-place notes ok")
    return True


if __name__ == "__main__":
    main()
