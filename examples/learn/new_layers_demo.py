"""AvgPool2d, ConvTranspose2d and LayerNorm1d shapes
(legacy/src/momijo/learn/examples/learn/new_layers_demo.mojo)."""
from momijo.tensor import tensor
from momijo.learn.nn.avgpool import AvgPool2d
from momijo.learn.nn.conv_transpose import ConvTranspose2d
from momijo.learn.nn.layernorm import LayerNorm1d


def main():
    x = tensor.randn([2, 3, 6, 6]).float()
    y = AvgPool2d((2, 2)).forward(x)
    print("AvgPool out:", y.shape())
    z = ConvTranspose2d(3, 2, (3, 3), (2, 2), (1, 1)).forward(x)
    print("Deconv out:", z.shape())
    out = LayerNorm1d(10).forward(tensor.randn([4, 10]).float())
    print("LayerNorm1d out:", out.shape())
    return y, z, out


if __name__ == "__main__":
    main()
