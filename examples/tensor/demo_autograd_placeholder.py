"""Reverse-mode gradients through the GradContext tape, checked against a numeric Jacobian
(mirrors legacy/examples/tensor/demo_autograd_placeholder.mojo and demo_autograd_jacobian_placeholder.mojo)."""
import momijo.tensor as mt
from momijo.tensor import autograd as ag


def main():
    ctx = ag.GradContext()
    w = ag.GradTensor.from_tensor(ctx, mt.from_list([1.0, -2.0, 3.0]), True)
    loss = w.square(ctx).mul(ctx, 0.5).sum_all(ctx)              # 0.5 * sum(w^2): gradient is w
    loss.backward(ctx)
    print("loss:", loss.item(ctx), "grad:", w.grad(ctx).tolist())
    assert w.grad(ctx).tolist() == [1.0, -2.0, 3.0]
    x0 = mt.from_list([1.0, 2.0])
    num, ana = mt.math.numeric_jacobian(mt.math.f_vec, x0), mt.math.analytic_jacobian(x0)
    assert mt.tensor.allclose(num, ana, atol=1e-5)
    return w.grad(ctx)


if __name__ == "__main__":
    main()
