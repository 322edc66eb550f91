"""The reference's method spellings on the dataframe classes: dtype tags, bitmaps, columns, typed series, the
multi-level index as levels + codes, aggregate tags and the frame's cell / column / row setters."""
import os

from momijo_b200.dataframe import ops as O
from momijo_b200.dataframe import relational as R
from momijo_b200.dataframe.frame import Bitmap, Column, DataFrame, DType, MultiIndex, Series, Value


def test_dtype_bitmap_column():
    d = DType.INT64(True)
    assert (d.tag, d.is_nullable(), d.is_int64(), DType.tag_f64()) == (3, True, True, 5) and not DType.STRING().is_nullable()
    b = Bitmap.from_mask([1, 0, 1])
    b.resize(5, True)
    assert str(b) == "Bitmap(10111)" and b.count_true() == 4 and not b.set(9, True) and len(b) == 5
    assert b.bit_and(Bitmap.all_false(5)).none_true() and b.bit_or(Bitmap.all_false(5)).to_mask() == b.to_mask()
    c = Column("a", [1, None, 3])
    assert (c.dtype(), c.dtype_name(), c.null_count(), c.value_str(0), c.value_str(1)) == (2, "i64", 1, "1", "")
    assert c.take([2, 9]).to_list() == [3, None] and c.gather(Bitmap.from_mask([1, 1, 0])).to_list() == [1, None]
    assert c.null_mask().values() == [False, True, False] and c.has_none() and not c.all_none()
    assert c.to_string(2) == "Column(name=a, dtype=i64, n=3, values=[1, None, ...])"
    assert Value.float64(2).as_string() == "2.0" and Value.bool(True).as_string() == "True"


def test_typed_series_and_pairs():
    s = R.SeriesI64([1, 2, None], "x")
    s.append(5)
    s.set(0, 7)
    assert s.values() == [7, 2, None, 5] and s.index() == [0, 1, 2, 3] and s.take([0, 10]).values() == [7, 0]
    assert s.head(2).values() == [7, 2] and s.count_valid() == 3 and abs(s.mean_as_f64() - 14 / 3) < 1e-12
    sb = R.SeriesBool([True, False, None])
    assert sb.logical_not().values() == [False, True, None] and sb.sum_true() == 1
    assert sb.logical_xor(R.SeriesBool([True, True, True])).values() == [False, True, None]
    ss = R.SeriesStr(["a", "b"])
    ss.resize(3)
    ss.set_null(0)
    assert ss.values() == [None, "b", None] and ss.null_count() == 2
    col = Column("c", [1])
    col.from_str(ss)
    assert col.dtype_name() == "str" and col.to_list() == [None, "b", None]
    cp = R.ColPair.of_i64("k", [1, 2])
    cp.push(3)
    assert cp.get(99) == "3" and cp.len() == 3 and R.ColPair.empty("e").is_empty()
    assert Series([1, 2], name="q").values() == [1, 2]


def test_multiindex_and_agg_tags():
    m = MultiIndex.from_arrays([["a", "a", "b"], ["x", "y", "x"]], ["k"])
    assert m.names == ["k", "level_1"] and m.levels_copy() == [["a", "b"], ["x", "y"]] and m.codes_copy() == [[0, 0, 1], [0, 1, 0]]
    assert m.values()[0] == "a\x1fx" and m.to_index_pair()[1] == "k,level_1" and m.is_lexsorted() and m.is_unique()
    assert m.take_rows([2, 0, 9]).tuples == [("b", "x"), ("a", "x")] and m.mask_rows([1, 0, 1]).nrows() == 2
    assert m.swaplevel(0, 1).tuples[1] == ("y", "a") and m.label_of(0, 1) == "y" and m.level_index_of(0, "q") == -1
    assert MultiIndex.from_product([["a", "b"], [1, 2]], ["u", "v"]).nrows() == 4
    a = O.Agg.parse("AVG")
    assert a.is_mean() and a.tag == 0 and O.Agg.max_("c").out == "c_max" and O.Agg.var_().name() == "var"
    e = R.Expr.both_and(R.Pred("a", R.Ops.GT, R.ConstVal.of_i64(1)), R.Pred("b", R.Ops.EQ, R.ConstVal.of_str("x")))
    assert e.kind == R.ExprKind.AND and e.left.pred.column == "a"
    assert R.ColumnBoolOps.between([1, 5, None, 3], 2, 5).bits == [False, True, False, True]


def test_frame_cells_columns_rows(tmp_path):
    df = DataFrame({"a": [1, 2, 2], "b": ["x", "y", "y"]})
    assert df.shape_str() == "(3, 2)" and df.find_col("b") == 1 and df.get_column("zz").len() == 0
    assert df.at(1, "b").get() == "y" and df.iat(5, 5).get() == "" and df.col_values("a") == ["1", "2", "2"]
    assert df.drop_duplicates(keep="last").index.labels == [0, 2] and df.with_rows(2).nrows() == 2
    assert df.assign({"c": lambda d: [v * 2 for v in d.col("a").values]}).col("c").values == [2, 4, 4]
    df.set_rows([True, False, False], "z")
    assert df.to_records()[0] == {"a": "z", "b": "z"} and df.set_iat(0, 0, Value(9)) and df.set_at(2, "b", "q") and not df.set_iat(9, 0, 1)
    assert df.to_string().splitlines()[:3] == ["DataFrame(3x2)", "a | b", "9 | z"]
    assert df.iloc(R.RowAll(), 0).to_list() == [9, 2, 2] and df.iloc([0, 2], [1]).to_records() == [{"b": "z"}, {"b": "q"}]
    assert df.loc([1], ["a"]).to_records() == [{"a": 2}] and df.index() == [0, 1, 2]
    other = DataFrame({"k": [5, 6, 7]})
    df.set_column("n", other)
    df.set_columns(["p", "q"], other)
    assert df.col_names() == ["a", "b", "n", "p", "q"] and df.col("q").values == [5, 6, 7]
    p = os.path.join(tmp_path, "x.csv")
    assert df.to_csv(p) and open(p).read().splitlines()[0] == "a,b,n,p,q"
    d2 = DataFrame()
    d2.from_series(Series([1, 2], name="s"))
    assert d2.to_records() == [{"s": 1}, {"s": 2}]
