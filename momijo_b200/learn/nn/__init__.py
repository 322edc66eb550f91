"""Layers (``momijo.learn.nn``)."""
from .module import Module, TAGS  # noqa: F401
from .layers import (  # noqa: F401
    Linear, ReLU, LeakyReLU, Sigmoid, Tanh, GELU, SiLU, BatchNorm1d, BatchNorm2d, Dropout, Flatten,
    QuantLinear, Embedding, LayerNorm, RMSNorm, RotaryEmbedding, SwiGLU, quantize_symmetric_int8,
    dropout_mask, Seq512,
)
from .conv import Conv2d, MaxPool2d  # noqa: F401
from .avgpool import AvgPool2d  # noqa: F401
from .conv_transpose import ConvTranspose2d  # noqa: F401
from .layernorm import LayerNorm1d  # noqa: F401
from .attention import MultiHeadAttention  # noqa: F401
from .transformer import EncoderLayer, DecoderLayer, TinyTransformer  # noqa: F401
from .rnn import GRU  # noqa: F401
from . import functional, activations, pool, init, regularizers  # noqa: F401
from ..api.sequential import Sequential as NNSequential  # noqa: F401,E402
