"""Tensors from nested Python lists of depth 1..4, dtype inferred from the literals
(legacy/examples/tensor/demo_build_from_literal_lists.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    v = mt.Tensor([1, 2, 3])
    m = mt.Tensor([[1.5, 2.0], [3.0, 4.5]])
    c = mt.Tensor([[[1, 0], [0, 1]], [[2, 2], [3, 3]]])
    q = mt.Tensor([[[[1.0]], [[2.0]]]])
    assert list(v.shape) == [3] and list(m.shape) == [2, 2] and list(c.shape) == [2, 2, 2] and list(q.shape) == [1, 2, 1, 1]
    assert not v.is_floating_point() and m.is_floating_point()
    assert mt.from_list_float32([1, 2, 3]).tolist() == [1.0, 2.0, 3.0]
    assert mt.from_2d_list_int([[1, 2], [3, 4]]).tolist() == [[1, 2], [3, 4]]
    assert mt.from_3d_list_float64([[[0.5]]]).tolist() == [[[0.5]]]
    assert m.tolist() == [[1.5, 2.0], [3.0, 4.5]]
    print("built", list(v.shape), list(m.shape), list(c.shape), list(q.shape))
    return 4


if __name__ == "__main__":
    main()
