"""Conv2d -> ReLU -> MaxPool2d -> Linear with explicit layer backward calls
(legacy/src/momijo/learn/examples/learn/train_cnn_backprop.mojo). The reference copies the pooled map
into a flat matrix element by element; here that is a reshape."""
from momijo.tensor import tensor
from momijo.learn.nn.conv import Conv2d, MaxPool2d
from momijo.learn.nn.layers import ReLU, Linear
from momijo.learn.losses.losses import softmax_cross_entropy, softmax
from momijo.learn.optim.sgd import SGD


def relu_backward(x, grad_y):
    pos = tensor.maximum_scalar(x, 0.0)
    return grad_y * (pos / (pos + 1e-12))


def main(epochs: int = 3):
    N, C, H, W = 16, 1, 16, 16
    conv = Conv2d(C, 4, (3, 3), (1, 1), (1, 1))
    relu, pool = ReLU(), MaxPool2d((2, 2), (2, 2))
    fc = Linear(4 * (H // 2) * (W // 2), 5)
    opt = SGD(0.05)
    x = tensor.randn([N, C, H, W]).float()
    y = softmax(tensor.randn([N, 5]))
    w = tensor.exp(y * 64.0)
    y = (w / tensor.matmul(w, tensor.ones([5, 1]))).float()   # sharpened to an almost one-hot target
    OH, OW = H // 2, W // 2
    losses = []
    for ep in range(epochs):
        h = conv.forward(x)
        a = relu.forward(h)
        p2 = pool.forward(a)
        flat = p2.reshape(N, 4 * OH * OW)
        logits = fc.forward(flat)
        loss, dlogits = softmax_cross_entropy(logits, y)
        dW2 = tensor.matmul(dlogits.transpose(), flat)
        db2 = tensor.matmul(dlogits.transpose(), tensor.ones([N, 1])).transpose()[0]
        dflat = tensor.matmul(dlogits, fc.weight)
        dp = dflat.reshape(N, 4, OH, OW)
        da = pool.backward(a, dp)
        dh = relu_backward(h, da)
        dW, db, _dx = conv.backward(x, dh)
        opt.step_linear(fc, dW2, db2)
        conv.weight.data = conv.weight.data - dW * opt.lr
        conv.bias_t.data = conv.bias_t.data - db * opt.lr
        print("epoch=", ep, " loss=", loss.item())
        losses.append(loss.item())
    probs = softmax(fc.forward(flat))
    print("probs shape:", probs.shape())
    return losses


if __name__ == "__main__":
    main()
