"""The method spellings of the reference on the learn classes: accessors, setters, builders, per-device layer
entry points and the summary table."""
import torch

import momijo_b200.learn as L
from momijo_b200.learn.amp.autocast import AMPPrecision, GradScaler, autocast
from momijo_b200.learn.data.dataset import Dataset, TupleDataset
from momijo_b200.learn.data.pair import Pair
from momijo_b200.learn.distributed.sharding import ShardRange, ZeroStage1
from momijo_b200.learn.distributed.strategies import DataParallel
from momijo_b200.learn.engine.jit_compile import JITOptions
from momijo_b200.learn.nn import BatchNorm2d, Conv2d, Dropout, Flatten, Linear, MaxPool2d
from momijo_b200.learn.nn.avgpool import AvgPool2d
from momijo_b200.learn.nn.conv_transpose import ConvTranspose2d
from momijo_b200.learn.optim import schedulers as S
from momijo_b200.learn.optim.adagrad import Adagrad
from momijo_b200.learn.optim.rmsprop import OptParam, RMSprop
from momijo_b200.learn.prob.distributions import Categorical, Normal
from momijo_b200.learn.utils.profiling import LabelProfiler, ScopedSection, ScopedTimer, Timer, TrainingLoopProfiler
from momijo_b200.learn.utils.randomness import RNG, SplitMix64, Xoshiro256ss
from momijo_b200.learn.utils.summary import model_summary


def test_data_containers():
    d = Dataset.from_list([1, 2, 3])
    d.insert(9, 4)
    d.set(0, 7)
    assert d.to_list() == [7, 2, 3, 4] and d.get(10, -1) == -1 and (d.front(), d.back()) == (7, 4)
    assert d.pop() == 4 and d.slice(-1, 2).to_list() == [7, 2] and not d.is_empty()
    t = TupleDataset.from_lists([1, 2, 3], [4, 5])
    t.append(9, 8)
    assert t.to_lists() == ([1, 2, 9], [4, 5, 8]) and t.get(7, 0, 0) == (0, 0)
    p = Pair.from_xy(torch.zeros(3, 4, 5), 2)
    assert (p.channels(), p.height(), p.width()) == (3, 4, 5) and p.is_valid() and str(p) == "Pair(shape=[3, 4, 5], y=2)"


def test_setters_and_builders():
    es = L.EarlyStopping(patience=1)
    es.set_mode("max")
    es.set_baseline(None)
    assert [es.on_epoch_end(0, 1.0), es.on_epoch_end(1, 0.5)] == [False, True] and "'stopped_epoch': 1" in es.summary()
    c = S.CosineAnnealingLR.__new__(S.CosineAnnealingLR)
    c.base_lr, c.min_lr = 1.0, 0.1
    c.set_base_lr(0.01)
    assert c.base_lr == 0.1
    c.set_min_lr(0.5)
    assert (c.base_lr, c.min_lr) == (0.5, 0.5)
    o = JITOptions()
    assert o.with_graph(True).graph and not o.graph
    a = autocast(False)
    assert not a.is_enabled() and a.enable().set_precision(AMPPrecision.fp16()).is_enabled() and not autocast.is_enabled()
    assert str(a) == "autocast(enabled=true, precision=fp16)" and not GradScaler(False).is_enabled()
    assert ShardRange(2, 5).clamp_index(9) == 5 and ShardRange(2, 5).length() == 3
    assert ZeroStage1(2, 1).shard_list_i32([1, 2, 3, 4, 5]) == [4, 5]
    dp = DataParallel(lambda x: x * 2, [0, 1], 2)
    assert dp.world_size() == 2 and dp.chunks() == 2 and dp(torch.ones(5, 1)).sum().item() == 10.0


def test_layer_entry_points_and_summary():
    lin = Linear(4, 3)
    lin.reset_parameters()
    x = torch.ones(2, 4)
    assert abs(lin.forward_auto(x)[0, 0].item() - 0.01) < 1e-7 and lin.forward_cpu_parallel(x).shape == (2, 3)
    assert [tuple(t.shape) for t in lin.backward_cpu_parallel(x, torch.ones(2, 3))] == [(3, 4), (3,), (2, 4)]
    if not torch.cuda.is_available():
        try:
            lin.forward_gpu(x)
            assert False
        except RuntimeError:
            pass
    assert Conv2d(1, 2, 3).forward_cpu_parallel(torch.ones(1, 1, 5, 5)).shape == (1, 2, 3, 3)
    assert MaxPool2d(2).backward_auto(torch.rand(1, 1, 4, 4), torch.ones(1, 1, 3, 3)).shape == (1, 1, 4, 4)
    assert Flatten().forward_cpu(torch.ones(2, 3, 4)).shape == (2, 12)
    assert AvgPool2d(2).backward(torch.rand(1, 1, 4, 4), torch.ones(1, 1, 2, 2)).flatten().tolist() == [0.25] * 16
    ct = ConvTranspose2d(2, 3, 3, (2, 2), (1, 1))
    xin = torch.rand(1, 2, 4, 4)
    assert tuple(ct(xin).shape[2:]) == ct.out_shape(4, 4) == (7, 7)
    text = model_summary(L.Sequential(Linear(4, 3), Dropout(), Flatten(), BatchNorm2d(3)))
    assert "Linear" in text and "[-1, 4] -> [-1, 3]" in text and text.rstrip().endswith("Total params: 21 | Trainable: 21 | Buffers: 6")


def test_optimizer_drivers_and_random_streams():
    r = RMSprop(lr=0.1)
    w, g = torch.ones(3), torch.full((3,), 0.5)
    r.set_params_tensor(w, g)
    r.step()
    r.zero_grad()
    assert w[0].item() < 1e-4 and g.tolist() == [0.0] * 3
    ps = [OptParam(1.0, 0.5)]
    r.set_params(ps)
    r.step()
    assert ps[0].value < 1e-4
    a = Adagrad(lr=0.1)
    assert abs(a.step_on_lists([1.0], [0.5])[0] - 0.9) < 1e-6 and abs(a.step_on_tensor_list([torch.ones(2)], [torch.full((2,), 0.5)])[0][0].item() - 0.9) < 1e-6
    a.reset_state()
    assert a.state == {}
    assert Categorical.from_probs_tensor(torch.tensor([1.0, -2.0, 3.0])).probs == [0.25, 0.0, 0.75] and Normal(2.0, 1.0).mean_value() == 2.0
    assert 0.0 < RNG.from_int_seed(-1).next_f64_open01() < 1.0 and SplitMix64(1).next() == 10451216379200822465
    assert Xoshiro256ss.from_seed(1).next_u64() == Xoshiro256ss(1).next_u64()


def test_profiling_call_forms():
    t = Timer()
    t.start(0)
    assert t.lap(5_000_000) == 0.005 and t.stop(1_000_000_000) == 1.0 and t.elapsed() == 1.0 and t.measure(10, 2_000_000_010) == 2.0
    p = TrainingLoopProfiler(4)
    p.begin_data(0)
    p.end_data(1_000_000)
    p.begin("forward", 5)
    p.end(2_000_005)
    assert p.summary()["forward"] == 2.0 and p.summary_lines()[0] == " - data: count=1, total_s=0.001, mean_s=0.001, sma_s=0.001"
    lp = LabelProfiler()
    lp.add_lap_s("x", 0.5)
    ScopedSection(lp, "y", 0).end(100)
    assert len(lp.summary()) == 2 and ScopedTimer(Timer(), 0).stop(3_000_000_000) == 3.0
