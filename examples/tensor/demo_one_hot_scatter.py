"""one_hot, gather, scatter and scatter-add (mirrors legacy/examples/tensor/demo_one_hot_scatter.mojo)."""
import momijo.tensor as mt


def main():
    labels = mt.from_list([2, 0, 1])
    hot = labels.one_hot(3)
    table = mt.from_list([[10.0, 11.0, 12.0], [20.0, 21.0, 22.0], [30.0, 31.0, 32.0]])
    picked = mt.gather(table, 1, labels.reshape(3, 1))
    placed = mt.scatter(mt.zeros([3, 3]), 1, labels.reshape(3, 1), mt.ones([3, 1]))
    counts = mt.zeros([3]).scatter_add_value(0, mt.from_list([0, 0, 2]), mt.ones([3]))
    print(hot.tolist(), picked.tolist(), placed.tolist(), counts.tolist())
    assert hot.tolist() == placed.tolist() and picked.reshape(3).tolist() == [12.0, 20.0, 31.0] and counts.tolist() == [2.0, 0.0, 1.0]
    return hot


if __name__ == "__main__":
    main()
