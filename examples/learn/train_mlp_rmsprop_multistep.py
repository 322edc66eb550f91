"""Two-layer MLP, hand-written backward, per-layer RMSprop and a multi-step schedule
(legacy/src/momijo/learn/examples/learn/train_mlp_rmsprop_multistep.mojo)."""
from momijo.tensor import tensor
from momijo.learn.nn.layers import Linear, ReLU
from momijo.learn.losses.losses import softmax_cross_entropy, softmax
from momijo.learn.optim.rmsprop import RMSprop
from momijo.learn.optim.scheduler_multistep import MultiStepLR


def main(epochs: int = 6):
    N, D, H, C = 64, 10, 32, 2
    l1, relu, l2 = Linear(D, H), ReLU(), Linear(H, C)
    opt = RMSprop(1e-2, alpha=0.9)
    sch = MultiStepLR(opt.lr, [2, 4], gamma=0.5)
    x = tensor.randn([N, D])
    y = softmax(tensor.randn([N, C]))
    losses = []
    for ep in range(epochs):
        a1 = relu.forward(l1.forward(x))
        logits = l2.forward(a1)
        loss, dlogits = softmax_cross_entropy(logits, y)
        dW2 = tensor.matmul(dlogits.transpose(), a1)
        db2 = tensor.matmul(dlogits.transpose(), tensor.ones([N, 1])).transpose()[0]
        da1 = tensor.matmul(dlogits, l2.weight)
        mask = tensor.maximum_scalar(a1, 0.0) / (tensor.maximum_scalar(a1, 0.0) + 1e-12)
        dh1 = da1 * mask
        dW1 = tensor.matmul(dh1.transpose(), x)
        db1 = tensor.matmul(dh1.transpose(), tensor.ones([N, 1])).transpose()[0]
        opt.step_linear(l2, dW2, db2)
        opt.step_linear(l1, dW1, db1)
        opt.lr = sch.step()
        print("epoch=", ep, " loss=", loss.item(), " lr=", opt.lr)
        losses.append(loss.item())
    return losses


if __name__ == "__main__":
    main()
