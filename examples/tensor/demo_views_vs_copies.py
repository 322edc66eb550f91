"""Which operations share storage with their source and which copy
(legacy/examples/tensor/demo_views_vs_copies.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    t = mt.arange_f32(0, 12).reshape(3, 4)
    views = [t[1], t[:, ::2], mt.transpose(t, 0, 1), mt.view(t, [4, 3]), mt.unsqueeze(t, 0)]
    for v in views:
        assert v.untyped_storage().data_ptr() == t.untyped_storage().data_ptr()
    copies = [t.clone(), mt.contiguous(mt.transpose(t, 0, 1)), t + 0.0, mt.flip(t, [0]), mt.cat([t, t], 0)]
    for c in copies:
        assert c.untyped_storage().data_ptr() != t.untyped_storage().data_ptr()
    t[1, 0] = -5.0
    assert views[0][0].item() == -5.0 and copies[0][1, 0].item() == 4.0
    print("views:", len(views), "copies:", len(copies))
    return len(views)


if __name__ == "__main__":
    main()
