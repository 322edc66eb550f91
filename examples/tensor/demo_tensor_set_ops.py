"""Sorted-unique set algebra on integer tensors (mirrors legacy/examples/tensor/demo_tensor_set_ops.mojo)."""
import momijo.tensor as mt


def main():
    a, b = mt.from_list([3, 1, 3, 2]), mt.from_list([2, 5, 2])
    u = mt.helpers.unique(a)
    print("unique:", u.values.tolist(), "counts:", u.counts.tolist())
    print("union:", a.set_union(b).tolist(), "intersection:", a.set_intersection(b).tolist())
    print("difference:", a.set_difference(b).tolist(), "xor:", a.set_xor(b).tolist(), "isin:", a.isin_(b).tolist())
    assert a.set_union(b).tolist() == [1, 2, 3, 5] and a.set_xor(b).tolist() == [1, 3, 5] and a.set_intersection(b).tolist() == [2]
    return u.values


if __name__ == "__main__":
    main()
