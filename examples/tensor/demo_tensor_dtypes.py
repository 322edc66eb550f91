"""dtype tags, casts between element types, the type-erased AnyTensor and complex scalars
(mirrors legacy/examples/tensor/demo_tensor_dtypes.mojo, demo_dtypes_devices_strides.mojo and
demo_types_bool_complex.mojo)."""
import momijo.tensor as mt


def main():
    x = mt.from_list([1.7, -2.2, 300.9])
    as_int, as_f32 = x.to_int(), x.to_float32()
    any_t = mt.AnyTensor(x)
    bytes_ = any_t.to_tensor_u8()
    z = mt.math.Complex128(1.0, 2.0) * mt.math.Complex128(0.0, 1.0)
    scalar = mt.cast.to_i8_from_f32(300.7)                       # wraps like a C cast
    print(as_int.tolist(), as_f32.dtype_name(), any_t.dtype.name, bytes_.tolist(), (z.real(), z.imag()), scalar)
    print("device:", mt.device.RuntimeDeviceContext.cpu().get(), "strides:", mt.zeros([2, 3, 4]).strides())
    assert as_int.tolist() == [1, -2, 300] and (z.real(), z.imag()) == (-2.0, 1.0) and scalar == 44
    return as_int


if __name__ == "__main__":
    main()
