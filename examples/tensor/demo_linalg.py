"""matmul, solve, inverse, QR / SVD / Cholesky and a tiny least-squares line fit
(mirrors legacy/examples/tensor/demo_linalg.mojo, demo_tensor_linalg.mojo and demo_tiny_linear_regression.mojo)."""
import momijo.tensor as mt


def main():
    a = mt.from_list([[4.0, 1.0], [1.0, 3.0]])
    b = mt.from_list([[1.0], [2.0]])
    x = mt.solve(a, b)
    q, r = mt.math.qr(a)
    u, s, vh = mt.math.svd(a)
    l = mt.math.cholesky(a)
    assert mt.tensor.allclose(mt.matmul(a, x), b) and mt.tensor.allclose(mt.matmul(q, r), a)
    assert mt.tensor.allclose(mt.matmul(l, mt.transpose(l)), a) and mt.tensor.allclose(mt.matmul(a, mt.inv(a)), mt.eye(2, dtype=a.dtype))
    xs = mt.from_list([[0.0, 1.0], [1.0, 1.0], [2.0, 1.0], [3.0, 1.0]])      # [x, 1] design matrix
    ys = mt.from_list([[1.0], [3.0], [5.0], [7.0]])                            # y = 2x + 1
    w = mt.solve(mt.matmul(mt.transpose(xs), xs), mt.matmul(mt.transpose(xs), ys))
    print("solve:", x.tolist(), "singular values:", s.tolist(), "det:", a.det(), "fit:", w.tolist())
    assert abs(w[0, 0].item() - 2.0) < 1e-5 and abs(w[1, 0].item() - 1.0) < 1e-5
    return w


if __name__ == "__main__":
    main()
