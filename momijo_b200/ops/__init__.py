"""Kernel front ends: GEMM, attention, normalisation, RoPE, activations, embedding, loss, optimizer."""
from .gemm import gemm, pick_bn  # noqa: F401
from .functional import (  # noqa: F401
    linear, mlp_gelu, swiglu, activation, layer_norm, rms_norm, rope_table, rope_inplace,
    attention_packed, embedding, softmax_cross_entropy, lm_head_cross_entropy, pad_vocab,
)
from .optim import adamw_flat, sgd_flat, sq_norm  # noqa: F401
