"""Boolean tensors and logic ops; complex numbers
(legacy/examples/tensor/demo_types_bool_complex.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    a = mt.Tensor([True, False, True])
    b = mt.Tensor([True, True, False])
    assert mt.and_t(a, b).tolist() == [1, 0, 0] or mt.and_t(a, b).tolist() == [True, False, False]
    assert mt.or_t(a, b).bool().tolist() == [True, True, True] and mt.xor_t(a, b).bool().tolist() == [False, True, True]
    assert mt.not_t(a).bool().tolist() == [False, True, False]
    assert mt.to_bool(mt.Tensor([0, 2, -1])).tolist() == [False, True, True]
    z = mt.complex(mt.Tensor([3.0, 0.0]), mt.Tensor([4.0, 1.0]))
    assert mt.complex_abs(z).tolist() == [5.0, 1.0]
    assert mt.complex_real(z).tolist() == [3.0, 0.0] and mt.complex_imag(z).tolist() == [4.0, 1.0]
    c = mt.Complex128(1.0, 2.0) * mt.Complex128(3.0, -1.0)
    assert (c.re, c.im) == (5.0, 5.0)
    print("bool / complex ok")
    return True


if __name__ == "__main__":
    main()
