"""Shapes that do not broadcast raise; the lenient mode of the reference is opt-in
(legacy/examples/tensor/demo_broadcast_trap.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a, b = mt.zeros([3, 4]), mt.zeros([5])
    try:
        a + b
        raised = False
    except Exception:
        raised = True
    assert raised
    try:
        mt.broadcast_shapes([2, 3], [4, 3, 2])
        ok = False
    except Exception:
        ok = True
    assert ok
    # a trailing singleton is the usual fix
    c = a + mt.zeros([3, 1])
    assert tuple(c.shape) == (3, 4)
    print("incompatible shapes raise; [3,4] + [3,1] ->", list(c.shape))
    return True


if __name__ == "__main__":
    main()
