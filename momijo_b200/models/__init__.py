"""Model families assembled from the kernel front ends."""
from .gpt2 import GPT2, GPT2Config  # noqa: F401
from .llama import Llama, LlamaConfig  # noqa: F401,E402
from .moe import MoEDecoder, MoEConfig  # noqa: F401,E402
