"""momijo.learn API family: the names re-exported by the reference's
``legacy/src/momijo/learn/__init__.mojo:10-184`` plus the additions the decoder configs need."""
from . import nn, losses, metrics, prob, optim, amp, data, distributed, engine, callbacks, profiler, utils, api, hub, audio, text  # noqa: F401

from .api.model import Model  # noqa: F401
from .api.sequential import Sequential, NNSequential, prepare, convert  # noqa: F401
from .api.functional import compile_model, fit, evaluate, predict  # noqa: F401
from .api.io import save_model, load_model  # noqa: F401
from .api.onnx_lite import export_onnx_lite  # noqa: F401
from .nn.module import Module  # noqa: F401
from .nn.layers import (  # noqa: F401
    Linear, ReLU, LeakyReLU, Sigmoid, Tanh, BatchNorm1d, BatchNorm2d, Dropout, Flatten, QuantLinear,
    Embedding, LayerNorm, RMSNorm, RotaryEmbedding, SwiGLU,
)
from .nn.conv import Conv2d, MaxPool2d  # noqa: F401
from .nn.avgpool import AvgPool2d  # noqa: F401
from .nn.conv_transpose import ConvTranspose2d  # noqa: F401
from .nn.layernorm import LayerNorm1d  # noqa: F401
from .nn.attention import MultiHeadAttention  # noqa: F401
from .nn.transformer import EncoderLayer, DecoderLayer, TinyTransformer  # noqa: F401
from .nn.rnn import GRU  # noqa: F401
from .nn.functional import conv2d, max_pool2d  # noqa: F401
from .nn.activations import relu, gelu, sigmoid, softmax, log_softmax  # noqa: F401
from .losses.classification import cross_entropy  # noqa: F401
from .losses.regression import mse_loss, mae_loss  # noqa: F401
from .losses.losses import softmax_cross_entropy, cross_entropy_from_logits, cross_entropy_from_probs  # noqa: F401
from .optim.sgd import SGD  # noqa: F401
from .optim.adam import Adam  # noqa: F401
from .optim.adamw import AdamW  # noqa: F401
from .optim.rmsprop import RMSprop  # noqa: F401
from .optim.adagrad import Adagrad  # noqa: F401
from .optim.scheduler_steplr import StepLR  # noqa: F401
from .optim.scheduler_multistep import MultiStepLR  # noqa: F401
from .optim.scheduler_cosine import CosineAnnealingLR  # noqa: F401
from .data.dataset import Dataset, IterableDataset, TupleDataset, TensorDataset  # noqa: F401
from .data.dataloader import DataLoader, DataLoaderOptions  # noqa: F401
from .data.sampler import RandomSampler, DistributedSampler  # noqa: F401
from .metrics.metrics import accuracy_approx  # noqa: F401
from .metrics.classification import accuracy, f1_score  # noqa: F401
from .metrics.regression import r2_score  # noqa: F401
from .callbacks.early_stopping import EarlyStopping  # noqa: F401
from .callbacks.model_checkpoint import ModelCheckpoint  # noqa: F401
from .callbacks.lr_monitor import LRMonitor  # noqa: F401
from .callbacks.logger import CSVLogger, CSVTableLogger  # noqa: F401
from .amp.autocast import autocast, GradScaler  # noqa: F401
from .engine.trainer import Trainer  # noqa: F401
from .engine.evaluator import Evaluator  # noqa: F401
from .engine.hooks import Hooks  # noqa: F401
from .engine.jit_compile import JITOptions, compile  # noqa: F401
from .profiler.core import Profiler  # noqa: F401
from .utils.profiling import TrainingLoopProfiler  # noqa: F401
from .utils.checkpoint import make_checkpoint, apply_checkpoint  # noqa: F401
from .utils.checkpoint_fileio import save_checkpoint_files, load_checkpoint_files  # noqa: F401
from .utils.tensor_bytes import pack_f64, unpack_f64  # noqa: F401
from .distributed.env import get_rank_world  # noqa: F401
from .distributed.ddp import ProcessGroup, init_process_group, destroy_process_group, DDPLinear  # noqa: F401
from .distributed import (  # noqa: F401
    DataParallel, DistributedDataParallel, ShardRange, partition_1d, ZeroStage1, ReduceOp,
    all_gather, reduce_scatter, all_to_all, send, recv, ShardedDataParallel,
)
from ..tensor import Tensor  # noqa: F401,E402
from ..tensor.autograd import GradContext, GradTensor, no_grad_begin, no_grad_end  # noqa: F401,E402

# Names that live in momijo_b200.parallel are resolved on first use: that package imports parts of this
# one (the collective facade), so importing it here at module load would be circular.
_PARALLEL_NAMES = {
    "ColumnParallelLinear": "tp", "RowParallelLinear": "tp", "VocabParallelEmbedding": "tp",
    "TopKRouter": "ep", "MoELayer": "ep", "PipelineStage": "pp", "Schedule1F1B": "pp",
    "ParallelConfig": "config", "HybridEngine": "engine",
}


def __getattr__(name):
    mod = _PARALLEL_NAMES.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib

    value = getattr(importlib.import_module(f"..parallel.{mod}", __name__), name)
    globals()[name] = value
    return value

from .. import _layout as _layout  # noqa: E402

_layout.link_siblings("learn")   # names the reference keeps in another file of this package still resolve
