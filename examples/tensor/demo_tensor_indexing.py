"""gather / scatter / take_along_axis / topk / argwhere
(legacy/examples/tensor/demo_tensor_indexing.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = np.array([[5.0, 1.0, 9.0], [2.0, 8.0, 3.0]])
    t = mt.Tensor(a.tolist())
    idx = mt.Tensor([[2, 0], [1, 1]]).long()
    assert mt.gather(t, 1, idx).tolist() == np.take_along_axis(a, np.array([[2, 0], [1, 1]]), 1).tolist()
    assert mt.take_along_axis(t, idx, 1).tolist() == mt.gather(t, 1, idx).tolist()
    z = mt.scatter(mt.zeros_f32([2, 3]), 1, idx, mt.Tensor([[1.0, 2.0], [3.0, 4.0]]))
    assert z.tolist() == [[2.0, 0.0, 1.0], [0.0, 4.0, 0.0]]
    vals, pos = mt.topk(t, 2)
    assert vals.tolist() == [[9.0, 5.0], [8.0, 3.0]] and pos.tolist() == [[2, 0], [1, 2]]
    assert mt.argwhere((t > 4).bool()).tolist() == np.argwhere(a > 4).tolist()
    print("tensor indexing ok")
    return True


if __name__ == "__main__":
    main()
