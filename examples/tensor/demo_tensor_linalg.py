"""matmul, solve, inverse, QR, Cholesky and SVD identities
(legacy/examples/tensor/demo_tensor_linalg.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    rng = np.random.default_rng(0)
    a = rng.normal(size=(4, 4)) + 4 * np.eye(4)
    b = rng.normal(size=(4, 2))
    A, B = mt.Tensor(a.tolist()).double(), mt.Tensor(b.tolist()).double()
    assert np.allclose(mt.matmul(A, B).tolist(), a @ b)
    x = mt.solve(A, B)
    assert np.allclose(mt.matmul(A, x).tolist(), b, atol=1e-8)
    assert np.allclose(mt.matmul(A, mt.inv(A)).tolist(), np.eye(4), atol=1e-8)
    q, r = mt.qr(A)
    assert np.allclose(mt.matmul(q, r).tolist(), a, atol=1e-8)
    spd = a @ a.T
    L = mt.cholesky(mt.Tensor(spd.tolist()).double())
    assert np.allclose(mt.matmul(L, mt.transpose(L, 0, 1)).tolist(), spd, atol=1e-8)
    u, s, vt = mt.svd(A)
    assert np.allclose((np.asarray(u.tolist()) * np.asarray(s.tolist())) @ np.asarray(vt.tolist()), a, atol=1e-8)
    print("linalg identities ok")
    return True


if __name__ == "__main__":
    main()
