"""Analytic op estimators (legacy/src/momijo/learn/profiler/estimators.mojo:10-17)."""


def est_ops_linear(n: int, fin: int, fout: int) -> float:
    return 2.0 * n * fin * fout


def est_ops_relu(n: int, d: int) -> float:
    return float(n * d)


def est_ops_attention(b: int, h: int, t: int, d: int, causal: bool = True) -> float:
    f = 4.0 * b * h * t * t * d
    return f / 2 if causal else f


def est_ops_conv2d(n, c, oc, oh, ow, kh, kw) -> float:
    return 2.0 * n * oc * oh * ow * c * kh * kw
