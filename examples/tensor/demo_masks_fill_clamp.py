"""Boolean masks: select, fill, where and clamp (mirrors legacy/examples/tensor/demo_masks_fill_clamp.mojo)."""
import momijo.tensor as mt


def main():
    x = mt.from_list([[-2.0, 5.0, 0.5], [9.0, -1.0, 3.0]])
    neg = x < 0.0
    picked = mt.indexing.masked_select(x, neg)
    filled = x.masked_fill_value(neg, 0.0)
    clipped = mt.clamp(x, 0.0, 4.0)
    labels = mt.where(x > 1.0, mt.ones([2, 3]), mt.zeros([2, 3]))
    print(picked.tolist(), filled.tolist(), clipped.tolist(), labels.tolist(), mt.indexing.argwhere(neg).tolist())
    assert picked.tolist() == [-2.0, -1.0] and clipped.max().item() == 4.0 and filled.min().item() == 0.0
    return clipped


if __name__ == "__main__":
    main()
