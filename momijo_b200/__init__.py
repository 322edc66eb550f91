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
from . import _layout as _layout  # noqa: F401,E402

_layout.install()       # reference module paths served from consolidated modules (``dataframe.series_bool`` ...)
