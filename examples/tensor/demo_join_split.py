"""cat / stack / chunk / split_sizes / unbind (mirrors legacy/examples/tensor/demo_join_split.mojo)."""
import momijo.tensor as mt


def main():
    a, b = mt.ones([2, 3]), mt.zeros([2, 3])
    rows = mt.cat([a, b], 0)
    planes = mt.stack([a, b], 0)
    halves = mt.chunk(rows, 2, 0)
    parts = rows.split_sizes([1, 3], 0)
    cols = mt.transform.unbind(a, 1)
    print(rows.shape, planes.shape, [tuple(h.shape) for h in halves], [tuple(p.shape) for p in parts], len(cols))
    assert tuple(rows.shape) == (4, 3) and tuple(planes.shape) == (2, 2, 3) and tuple(parts[1].shape) == (3, 3) and len(cols) == 3
    return rows


if __name__ == "__main__":
    main()
