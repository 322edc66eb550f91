"""CPU tests of the momijo.tensor API family: NumPy-parity indexing / setitem, promotion rules,
seeded factories, autograd compat, dtype lattice, text I/O."""
import numpy as np
import pytest
import torch

import momijo_b200.tensor as T


def test_promotion_rules():
    a = T.from_list_int([1, 2, 3, 4], [2, 2])
    assert (a + a).dtype == torch.int64 and (a * 2).dtype == torch.int64
    assert (a / a).dtype == torch.float64 and (a % 2).dtype == torch.float64
    assert (a @ a).dtype == torch.float32
    f32 = T.from_list_float32([1.0, 2.0])
    assert (f32 + T.from_list_int([1, 2])).dtype == torch.float32
    assert (f32 + T.from_list_float64([1.0, 2.0])).dtype == torch.float64
    m = a > 2
    assert m.dtype == torch.int64 and m.tolist() == [[0, 0], [1, 1]]
    assert T.where(m, a, T.zeros_like(a)).tolist() == [[0, 0], [3, 4]]


@pytest.mark.parametrize("spec,key", [
    ("1", 1), ("-1", -1), ("1:3", slice(1, 3)), ("::2", slice(None, None, 2)), ("::-1", slice(None, None, -1)),
    ("0, :", (0, slice(None))), (":, 1:3", (slice(None), slice(1, 3))), ("1, 2, ::2", (1, 2, slice(None, None, 2))),
    ("..., 0", (Ellipsis, 0)), (":, None, 1", (slice(None), None, 1)),
])
def test_indexing_numpy_parity(spec, key):
    n = np.arange(60).reshape(3, 4, 5)
    t = T.from_list_int(n.tolist())
    assert np.array_equal(np.asarray(t[T.S(spec)].tolist()), n[key])
    assert np.array_equal(np.asarray(t[key].tolist()), n[key])


def test_setitem_numpy_parity_1d_to_5d():
    for nd in range(1, 6):
        shape = [2, 3, 2, 3, 2][:nd]
        n = np.zeros(shape)
        t = T.zeros(shape)
        key = tuple([slice(0, 1)] + [slice(None)] * (nd - 1))
        n[key] = 7
        t[key] = 7
        n[..., -1] = -1
        t[T.S("..., -1")] = -1
        assert np.array_equal(np.asarray(t.tolist()), n)


def test_seeds_and_determinism():
    assert T.to_string(T.randn([3], seed=5)) == T.to_string(T.randn([3], seed=5))
    assert T.to_string(T.randn([3], seed=5)) != T.to_string(T.randn([3], seed=6))
    assert T.randperm_int(10, seed=1).tolist() == T.randperm_int(10, seed=1).tolist()
    assert T.zeros_f32([2]).dtype == torch.float32 and T.eye_int(2).tolist() == [[1, 0], [0, 1]]
    assert T.linspace_f64(0, 1, 5).tolist() == [0.0, 0.25, 0.5, 0.75, 1.0] and T.arange(3).dtype == torch.float32


def test_autograd_compat_and_single_visit():
    ctx = T.GradContext()
    x = T.GradTensor.from_tensor(ctx, T.from_list_float32([1.0, 2.0, 3.0]), True)
    y = x.mul(ctx, x)                       # reachable by two paths: gradient must be 2x, not 4x
    y.sum_all(ctx).backward(ctx)
    assert x.grad(ctx).tolist() == [2.0, 4.0, 6.0]
    T.no_grad_begin(ctx)
    z = x.exp(ctx)
    T.no_grad_end(ctx)
    assert not z.requires_grad and x.relu(ctx).requires_grad
    ctx2 = T.GradContext()
    lg = T.GradTensor.from_tensor(ctx2, T.from_2d_list_float32([[1.0, 2.0, 0.5], [0.1, 0.2, 3.0]]), True)
    loss = T.autograd.cross_entropy(ctx2, lg, T.from_list_int([1, 2]))
    ref = torch.nn.functional.cross_entropy(torch.tensor([[1.0, 2.0, 0.5], [0.1, 0.2, 3.0]]), torch.tensor([1, 2]))
    assert abs(float(loss.value()) - float(ref)) < 1e-6
    b = T.autograd.bce_with_logits(ctx2, lg, T.zeros([2, 3]))
    assert abs(float(b.value()) - float(torch.nn.functional.binary_cross_entropy_with_logits(lg.value(), torch.zeros(2, 3)))) < 1e-6


def test_dtype_lattice():
    f = T.from_name
    assert T.promote_dtype(f("bool"), f("uint8")).name == "uint8"
    assert T.promote_dtype(f("int32"), f("float16")).name == "float16"
    assert T.promote_dtype(f("float16"), f("bfloat16")).name == "float32"
    assert T.promote_dtype(f("float32"), f("float64")).name == "float64"
    assert T.can_cast(f("int32"), f("float64")) and not T.can_cast(f("float32"), f("int32"))
    assert T.can_cast(f("float32"), f("int32"), "unsafe") and T.from_code(T.to_code(f("int16"))).itemsize == 2


def test_text_io_and_transforms(tmp_path):
    x = T.from_2d_list_float64([[1.5, -2.0], [3.25, 4.0]])
    for w, r, ext in [(T.write_csv_f64, T.read_csv_f64, "csv"), (T.write_json_f64, T.read_json_f64, "json"),
                      (T.write_xml_f64, T.read_xml_f64, "xml")]:
        p = str(tmp_path / f"t.{ext}")
        assert w(x, p) and r(p).tolist() == x.tolist()
    xi = T.from_list_int([1, 2, 3])
    p = str(tmp_path / "i.csv")
    T.write_csv_int(xi, p)
    assert T.read_csv_int(p).reshape(-1).tolist() == [1, 2, 3]
    assert T.pad(T.arange_f32(3), [(2, 1)], "symmetric").tolist() == [1, 0, 0, 1, 2, 2]
    assert T.pad(T.arange_f32(3), [(1, 1)], "circular").tolist() == [2, 0, 1, 2, 0]
    assert T.matmul(T.ones_f32([2, 3]), T.ones_f32([3])).tolist() == [3.0, 3.0]
    with pytest.raises(T.TensorError):
        T.matmul(T.ones_f32([2, 3]), T.ones_f32([2, 2]))
    with T.compat.lenient():
        assert T.matmul(T.ones_f32([2, 3]), T.ones_f32([2, 2])).numel() == 0
    a = T.from_list_int([3, 1, 2, 3])
    assert a.unique_().tolist() == [1, 2, 3] and a.union(T.from_list_int([9])).tolist() == [1, 2, 3, 9]
    assert a.one_hot(4).tolist()[0] == [0, 0, 0, 1] and a.nanmin().item() == 1
