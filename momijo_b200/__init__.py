"""momijo_b200: a Blackwell-native deep-learning framework with momijo's capabilities.

Sub-packages
  tensor, learn, dataframe, vision, visual : the public API families of momijo
  ops      : front ends of the hand-written sm_100a kernels
  models   : GPT-2, Llama and MoE decoders built from those ops
  parallel : process groups, peer-memory runtime, DDP / ZeRO / TP / EP / PP
  utils    : timing, clocks, checkpoint blobs
"""
__version__ = "0.1.0"

from . import _C  # noqa: F401
