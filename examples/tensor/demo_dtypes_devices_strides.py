"""dtype names and sizes, device placement, strides of views
(legacy/examples/tensor/demo_dtypes_devices_strides.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    t = mt.arange_f32(0, 24).reshape(2, 3, 4)
    assert t.stride() == (12, 4, 1) and t.is_contiguous()
    p = mt.permute(t, [2, 0, 1])
    assert p.stride() == (1, 12, 4) and not p.is_contiguous()
    assert mt.contiguous(p).stride() == (6, 3, 1)
    i8 = mt.astype(t, "int8")
    f64 = mt.to_float64(t)
    assert i8.element_size() == 1 and f64.element_size() == 8
    assert mt.promote_dtype(mt.from_name("int32"), mt.from_name("float32")).name == "float32"
    d = mt.device_of(t)
    assert str(d).lower().startswith("cpu") or "cpu" in repr(d).lower()
    print("strides", t.stride(), p.stride(), "device", d)
    return t.stride()


if __name__ == "__main__":
    main()
