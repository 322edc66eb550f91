"""Linear -> BatchNorm1d -> ReLU -> Dropout -> Linear in a Sequential
(legacy/src/momijo/learn/examples/learn/sequential_full.mojo)."""
from momijo.tensor import tensor
from momijo.learn.nn.layers import Linear, ReLU, BatchNorm1d, Dropout
from momijo.learn.nn.module import Module
from momijo.learn.api.sequential import Sequential


def main():
    net = Sequential()
    net.add(Module.from_linear(Linear(10, 32)))
    net.add(Module.from_batchnorm1d(BatchNorm1d(32)))
    net.add(Module.from_relu(ReLU()))
    net.add(Module.from_dropout(Dropout(0.2)))
    net.add(Module.from_linear(Linear(32, 2)))
    x = tensor.randn([4, 10])
    y = net.forward(x)
    print("y shape:", y.shape())
    return y


if __name__ == "__main__":
    main()
