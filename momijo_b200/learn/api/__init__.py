"""High-level API (``momijo.learn.api``)."""
from .model import Model, CompileConfig  # noqa: F401
from .sequential import Sequential, NNSequential, QConfig, MinMaxObserver, Prepared, Converted, prepare, convert, get_default_qconfig  # noqa: F401
from .functional import (  # noqa: F401
    compile_model, fit, fit_with_options, evaluate, evaluate_with_options, predict, predict_with_options, FitOptions, FitResult, EvalOptions,
    PredictOptions, quantize_symmetric_int8, matmul_i8_i8_to_i32, dequantize_i32_to_f32_add_bias,
)
from .io import save_model, save_model_ok, load_model, load_model_ok, load_into  # noqa: F401
from . import serialization  # noqa: F401
from .serialization import save, load, save_linear, load_linear  # noqa: F401
from .onnx_lite import export_onnx_lite, emit_onnx_lite  # noqa: F401
