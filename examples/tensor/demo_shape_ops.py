"""reshape / transpose / permute / squeeze / unsqueeze / flatten and which of them share storage
(mirrors legacy/examples/tensor/demo_shape_ops.mojo, demo_reshape.mojo and demo_views_vs_copies.mojo)."""
import momijo.tensor as mt


def main():
    x = mt.arange(0, 24).reshape(2, 3, 4)
    t = mt.transpose(x, 0, 2)
    p = mt.permute(x, [1, 0, 2])
    s = mt.squeeze(mt.unsqueeze(x, 0), 0)
    f = mt.flatten(x, 1)
    inferred = x.reshape_infer([-1, 6])
    view = x[0]
    view[0, 0] = 99                     # a basic index is a view: the write shows in x
    clone = x.copy()
    clone[0, 0, 0] = -1                 # a copy owns its storage
    print(t.shape, p.shape, s.shape, f.shape, inferred.shape, x.strides(), t.is_contig())
    assert x[0, 0, 0].item() == 99 and tuple(f.shape) == (2, 12) and tuple(inferred.shape) == (4, 6) and not t.is_contig()
    return x


if __name__ == "__main__":
    main()
