"""Spot checks of the tensor package's smaller public names (casts, typed factories, op-id dispatchers, index
arithmetic, reductions, padding index maps, text I/O, tape record)."""
import math

import torch

from momijo_b200.tensor import (autograd as A, axis as AX, broadcast as B, cast as C, creation as CR, errors as E,
                                from_list, helpers as H, indexing as I, io as IO, math as M, nanops as N,
                                tensor as TT, transform as T, zeros)
from momijo_b200.tensor.gpu import runtime as R


def test_scalar_casts_follow_one_rule():
    assert C.to_i8_from_f32(300.7) == 44 and C.to_u8_from_f64(-1.0) == 255 and C.to_i32_from_f64(float("nan")) == 0
    assert C.to_f32_from_f64(0.1) == 0.10000000149011612 and C.to_f16_from_f32(1e6) == math.inf
    assert C.f32_to_int8(-129.9) == 127 and C.id_f32(5) == 5 and C.opt_i_to_f64(None) is None
    assert C.to_bool_from_f32(0.0) is False and C.to_int_from_float32(2.9) == 2


def test_typed_factories():
    assert CR.arange_u8(2, 5).tolist() == [2, 3, 4] and CR.arange_i32(3).dtype == torch.int32
    assert sorted(CR.randperm_u16(5, 3).tolist()) == [0, 1, 2, 3, 4]
    assert CR.randu_f32([4], 1.0, 2.0, 7).tolist() == CR.randu_f32([4], 1.0, 2.0, 7).tolist()
    assert CR.arange_with(3, lambda v: v * 2).tolist() == [0, 2, 4] and CR.linspace_Int(0, 10, 3).tolist() == [0, 5, 10]
    assert CR.rotl64(1, 65) == 2 and CR.linspace_list_f64(0, 1, 2, False) == [0.0, 0.5]


def test_op_id_dispatchers_and_logic():
    x, i = from_list([-1.5, 0.0, 2.5]), from_list([1, 0, 3])
    assert M.apply_unary(x, 13).tolist() == [-2.0, 0.0, 3.0] and M.apply_unary(i, 2).dtype == torch.float64
    assert M.land_t(x, i).tolist() == [True, False, True] and M.lnot_t(i).tolist() == [False, True, False]
    assert M.mod_t(from_list([5, 7]), from_list([3, 4])).tolist() == [2, 3]
    y = from_list([1.0, 2.0, 3.0])
    M.iadd_t(y, x)
    assert y.tolist() == [-0.5, 2.0, 5.5]
    assert M.round64(-2.5) == -3.0 and abs(M.selu64(-1.0) + 1.1113307378125625) < 1e-12
    J = M.numeric_jacobian(M.f_vec, from_list([1.0, 2.0]))
    assert torch.allclose(torch.tensor(J.tolist()), torch.tensor(M.analytic_jacobian(from_list([1.0, 2.0])).tolist()), atol=1e-6)
    assert B.bin32(2, 3, 4) == 8.0 and B.u64(-1, 6) == 0.0 and B.pow_generic_safe(2, 10) == 1024
    o = zeros([2])
    B.add_(from_list([1.0, 2.0]), from_list([3.0, 4.0]), o)
    assert o.tolist() == [4.0, 6.0]


def test_index_arithmetic_and_selectors():
    assert H.unravel_index(7, [2, 4]) == [1, 3] and H.lin_index([1, 3], [4, 1]) == 7
    assert H.range_len(0, 10, 3) == 4 and H.range_len(10, 0, -3) == 4 and H.compute_new_shape([2, 3], [(1, 1), (0, 2)]) == [4, 5]
    idx, n = [0, 0], 1
    while H.index_advance(idx, [2, 3]):
        n += 1
    assert n == 6
    u = H.unique(from_list([3, 1, 3, 2]))
    assert u.values.tolist() == [1, 2, 3] and u.counts.tolist() == [1, 1, 2]
    assert H.histogram_int(from_list([1, 2, 3, 4, 5]), [1, 3, 5]).counts.tolist() == [2, 3]
    picked = H.select(from_list([[1, 2, 3], [4, 5, 6]]), [H.make_index_sel(1), H.make_fancy_sel([0, 2])])
    assert picked.tolist() == [4, 6]
    x = from_list([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0], [7.0, 8.0, 9.0]])
    assert I.band(x, 0, 1).tolist() == [[1, 2, 0], [0, 5, 6], [0, 0, 9]] and I.at(x, 1, 2) == 6.0
    y = zeros([2, 2])
    I.fill_diagonal(y, 5.0)
    I.put(y, [1], [9.0])
    assert y.tolist() == [[5.0, 9.0], [0.0, 5.0]]
    c = zeros([3, 3])
    assert I.sgemm_contig_kernel_base(x, x, c, 1.0, 0.0) and c.tolist()[0] == [30.0, 36.0, 42.0]
    assert I.norm_range(0, 10, 3, 5) == [0, 3] and list(I.NDLinearIter([2, 2], [2, 1], 3)) == [3, 4, 5, 6]
    base = torch.arange(12.0)
    assert TT.share(base, [2, 3], [6, 1], 1).tolist() == [[1, 2, 3], [7, 8, 9]]


def test_reductions_padding_io_tape(tmp_path):
    x = from_list([[1.0, float("nan"), 3.0], [4.0, 5.0, 6.0]])
    assert AX.nan_sum(x, axis=1).tolist() == [4.0, 15.0] and AX.nanargmax(x, axis=1).tolist() == [2, 2]
    assert AX.quantile_1d_partial([1, 2, 3, 4], 0.5) == 2.5 and AX.select_kth([5, 1, 4, 2], 2) == 4
    assert AX.shape_drop_axes([2, 3, 4], [-1, 0]) == [3] and AX.unique(from_list([3, 1, 3])).tolist() == [3, 1]
    assert [T.reflect_index(i, 4) for i in range(-3, 7)] == [3, 2, 1, 0, 1, 2, 3, 2, 1, 0]
    assert [T.symmetric_index(i, 3) for i in range(-3, 6)] == [2, 1, 0, 0, 1, 2, 2, 1, 0]
    assert T.pad1d(from_list([1, 2]), 1, 2, 9).tolist() == [9, 1, 2, 9, 9]
    assert T.pad_nd_map(from_list([1, 2, 3]), [(2, 2)], 1).tolist() == [3, 2, 1, 2, 3, 2, 1]
    assert T.view_reshape_strides_if_contiguous([2, 6], [3, 4]) == (True, [4, 1])
    m = from_list([[1.5, 2.0], [3.0, 4.0]])
    for back in (IO.csv_to_tensor_with(IO.tensor_to_csv(m)), IO.json_numbers_to_tensor_with(IO.tensor_to_json_array(m)),
                 IO.xml_numbers_to_tensor_with(IO.tensor_to_xml_numbers(m))):
        assert back.tolist() == m.tolist()
    p = str(tmp_path / "m.csv")
    assert IO.write_csv(m, None, p) and IO.read_csv_with(p).tolist() == m.tolist()
    assert N.nan_to_num_f64(float("nan")) == 0.0 and N.nanmin_all_f64(from_list([float("nan"), 2.0])) == 2.0
    assert E.check_product([2, 3], 6) and not E.check_axis_status(3, 2).ok
    t = A.Tape()
    leaf = t.add_leaf(from_list([1.0, 2.0]))
    node = t.add_node(from_list([2.0, 4.0]), A.TAG_MULS(), leaf, s=2.0)
    assert len(t) == 2 and t.parents[node] == [0, -1] and A.TAG_WHERE() == 90
    w, mm, vv = [1.0], [0.0], [0.0]
    R.launch_adam_1d_cpu(w, [0.1], mm, vv, 0.1, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001)
    assert abs(w[0] - 0.9) < 1e-6


def test_tensor_method_spellings_and_cursors():
    from momijo_b200.tensor import Tensor
    from momijo_b200.tensor import device as D, dtype as DT
    from momijo_b200.tensor.tensor_dyn import AnyBuffer, AnyTensor
    x = from_list([[1, 2, 3], [4, 5, 6]])
    assert x.select_copy([x.idx(1)]).tolist() == [4, 5, 6] and x.select_view([x.all_axis(), x.slc(0, 3, 2)]).tolist() == [[1, 3], [4, 6]]
    x.select_set_scalar([x.idx(0), x.rng(1, 3)], 9)
    assert x.tolist() == [[1, 9, 9], [4, 5, 6]] and x.slice([(0, 2, 1), (1, 3, 1)]).tolist() == [[9, 9], [5, 6]]
    assert x.get2(1, 2) == 6 and x.len() == 2 and x.slice_inplace(1, 2, None, -1).tolist() == [[9, 9, 1], [6, 5, 4]]
    b = Tensor([0.0])
    b.append(1.0); b.append_list([2.0, 3.0]); b.append_repeat(7.0, 2); b.set_shape_row_major([2, 3])
    assert b.tolist() == [[0.0, 1.0, 2.0], [3.0, 7.0, 7.0]]
    assert x.not_bitwise().sum().item() == 0 and x.lshift_scalar(1).tolist()[1] == [8, 10, 12] and x.mod_scalar(4).tolist()[1] == [0, 1, 2]
    assert x.set_xor(from_list([9, 100])).tolist() == [1, 4, 5, 6, 100] and x.can_broadcast_with(from_list([1, 2, 3])) and not x.can_broadcast_with(from_list([1, 2, 3]), True)
    it = I.NDIter([2, 2])
    assert it.next() == (True, [0, 0]) and it.next() == (True, [0, 1]) and list(I.NDIter([])) == [[]]
    lin = I.NDLinearIter([2, 2], [2, 1], 1)
    assert lin.next() == (True, [0, 0], 1) and lin.next() == (True, [0, 1], 2)
    st = E.ErrStatus(E.ErrorKind.OutOfBounds(), "axis 3", "check_axis")
    assert st.ravel() == "[OutOfBounds] axis 3 (at check_axis)" and st.is_err() and E.ErrorKind.SHAPE == 2
    assert E.Err(E.ErrorKind.DivideByZero, "x").unwrap_or(5) == 5 and E.Ok(3).unwrap_or(5) == 3
    ctx = A.GradContext()
    g = A.GradTensor.from_tensor(ctx, from_list([1.0, -2.0]), True)
    assert g.shape(ctx) == [2] and g.at_flat(ctx, 1) == -2.0 and g.gt_scalar(ctx, 0.0).to_list(ctx) == [1.0, 0.0]
    assert g.select(ctx, from_list([1, 0]), g.mul(ctx, 2.0)).to_list(ctx) == [1.0, -4.0] and g.value(ctx).tolist() == [1.0, -2.0]
    a = AnyTensor(from_list([1.5, 2.5]))
    assert a.to_tensor_i32().tolist() == [1, 2]
    a.full_like_dtype_shape(DT.from_name("int32"), [2], 3.9)
    assert a.unwrap().tolist() == [3, 3]
    buf = AnyBuffer()
    buf.append_cast_from_f64(3.7, DT.from_name("int32").tag)
    assert buf.length() == 1 and buf.get_f64(0) == 3.0
    c = D.RuntimeDeviceContext.cpu()
    assert c.get().is_cpu() and CR.RNG64(1).next_i32(3, 4) == 3
