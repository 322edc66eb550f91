"""The hand-written training loop: forward, softmax cross-entropy with its gradient, manual backward
through two Linear layers, per-layer SGD (legacy/src/momijo/learn/examples/learn/train_full.mojo)."""
from momijo.tensor import tensor
from momijo.learn.nn.layers import Linear, ReLU
from momijo.learn.losses.losses import softmax_cross_entropy, softmax
from momijo.learn.optim.sgd import SGD


def main(epochs: int = 3):
    N, D, H, C = 64, 10, 32, 2
    l1, relu, l2, opt = Linear(D, H), ReLU(), Linear(H, C), SGD(0.1)
    x = tensor.randn([N, D])
    r = tensor.randn([N, 1])
    p = tensor.exp(r) / (tensor.exp(r) + tensor.exp(-r))
    q = p - (tensor.zeros([N, 1]) + 0.5)
    ind1 = tensor.maximum_scalar(q, 0.0) / (tensor.maximum_scalar(q, 0.0) + 1e-12)
    ind0 = 1.0 - ind1
    y = tensor.concat([ind0, ind1], axis=1)
    losses = []
    for ep in range(epochs):
        h1 = l1.forward(x)
        a1 = relu.forward(h1)
        logits = l2.forward(a1)
        loss, dlogits = softmax_cross_entropy(logits, y)
        onesN = tensor.ones([N, 1])
        dW2 = tensor.matmul(dlogits.transpose(), a1)
        db2 = tensor.matmul(dlogits.transpose(), onesN).transpose()[0]
        da1 = tensor.matmul(dlogits, l2.weight)
        mask = tensor.maximum_scalar(a1, 0.0) / (tensor.maximum_scalar(a1, 0.0) + 1e-12)
        dh1 = da1 * mask
        dW1 = tensor.matmul(dh1.transpose(), x)
        db1 = tensor.matmul(dh1.transpose(), onesN).transpose()[0]
        opt.step_linear(l2, dW2, db2)
        opt.step_linear(l1, dW1, db1)
        print("epoch=", ep, " loss=", loss.item())
        losses.append(loss.item())
    probs = softmax(l2.forward(relu.forward(l1.forward(x))))
    print("probs shape:", probs.shape())
    return losses


if __name__ == "__main__":
    main()
