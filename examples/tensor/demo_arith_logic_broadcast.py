"""Arithmetic with scalars and tensors, comparisons, logical ops and the broadcasting rule, including the
shape trap of a column against a row (mirrors legacy/examples/tensor/demo_arith_logic_broadcast.mojo,
demo_broadcast_align.mojo and demo_broadcast_trap.mojo)."""
import momijo.tensor as mt


def main():
    col = mt.from_list([[1.0], [2.0], [3.0]])
    row = mt.from_list([[10.0, 20.0]])
    grid = col + row                                   # (3,1) + (1,2) -> (3,2): often a surprise
    scaled = col.mul_scalar(2.0).add_scalar(1.0)
    mask = (grid > 21.0)
    both = mt.math.land_t(mask, grid < 23.0)
    print(grid.tolist(), scaled.tolist(), both.tolist(), mt.broadcast_shapes([3, 1], [1, 2]))
    assert tuple(grid.shape) == (3, 2) and col.can_broadcast_with(row) and not col.can_broadcast_with(mt.zeros([2, 2]))
    assert both.tolist() == [[False, False], [False, True], [False, False]]
    return grid


if __name__ == "__main__":
    main()
