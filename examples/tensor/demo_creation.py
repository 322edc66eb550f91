"""Factories: zeros / ones / full / arange / linspace / eye, seeded random tensors and typed variants
(mirrors legacy/examples/tensor/demo_creation.mojo and demo_build_from_literal_lists.mojo)."""
import momijo.tensor as mt


def main():
    z, o, f = mt.zeros([2, 3]), mt.ones([2, 3]), mt.full([2, 2], 7.5)
    r = mt.arange(0, 10, 2)
    ls = mt.creation.linspace_f64(0.0, 1.0, 5)
    e = mt.eye(3)
    g1, g2 = mt.randn([2, 2], seed=42), mt.randn([2, 2], seed=42)
    lit = mt.from_list([[1, 2, 3], [4, 5, 6]])
    u8 = mt.creation.arange_u8(2, 5)
    print(z.shape, o.sum().item(), f.tolist(), r.tolist(), ls.tolist(), e.trace().item(), lit.dtype_name(), u8.tolist())
    assert g1.tolist() == g2.tolist() and lit.shape_list() == [2, 3] and ls.tolist()[1] == 0.25
    return lit


if __name__ == "__main__":
    main()
