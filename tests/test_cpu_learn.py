"""CPU tests of the momijo.learn API family: closed-form schedulers, GradScaler state machine,
partition_1d / DistributedSampler, MNP round trips, streaming-metric merge, Trainer contract."""
import json
import math
import os

import pytest
import torch

import momijo_b200.learn as L
from momijo_b200.learn.optim import schedulers as S
from momijo_b200.learn.data.sampler import _assert_dist_shapes_equal


def test_partition_1d_balanced():
    for total in (0, 1, 10, 103):
        for world in (1, 2, 3, 8):
            rs = [L.partition_1d(total, world, r) for r in range(world)]
            assert rs[0].start == 0 and rs[-1].end == total
            assert all(a.end == b.start for a, b in zip(rs, rs[1:]))
            sizes = [r.size() for r in rs]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_distributed_sampler_reference_semantics():
    assert _assert_dist_shapes_equal(4, 103, False) and _assert_dist_shapes_equal(4, 103, True)
    W, n = 4, 10
    parts = [L.DistributedSampler(n, W, r, shuffle=True, seed=7, drop_last=False).epoch_indices(3) for r in range(W)]
    flat = sorted(i for p in parts for i in p)
    assert len(flat) == 12 and set(flat) == set(range(n))      # padded by repeating from the start
    parts = [L.DistributedSampler(n, W, r, drop_last=True).epoch_indices(0) for r in range(W)]
    assert all(len(p) == 2 for p in parts) and len({i for p in parts for i in p}) == 8
    a = L.DistributedSampler(n, 2, 0, seed=1).epoch_indices(0)
    assert a == L.DistributedSampler(n, 2, 0, seed=1).epoch_indices(0)
    assert a != L.DistributedSampler(n, 2, 0, seed=1).epoch_indices(1)


def test_schedulers_closed_form():
    s = S.StepLR(1.0, 3, 0.1)
    assert s.get_lr() == 1.0
    assert [round(s.step(), 6) for _ in range(7)] == [1, 1, 1, 0.1, 0.1, 0.1, 0.01]
    e = S.ExponentialLR(2.0, 0.5)
    assert [e.step() for _ in range(3)] == [2.0, 1.0, 0.5]
    m = S.MultiStepLR(1.0, [2, 4], 0.1)
    assert [round(m.step(), 6) for _ in range(5)] == [1, 1, 0.1, 0.1, 0.01]
    p = S.PolynomialLR(1.0, 4, power=2.0, min_lr=0.0)
    assert abs(p.step_to(2) - 0.25) < 1e-12 and p.step_to(9) == 0.0
    c = S.CosineAnnealingLR(1.0, 10, 0.1)
    assert abs(c.step_to(5) - (0.1 + 0.45 * (1 + math.cos(math.pi / 2)))) < 1e-12
    wr = S.CosineAnnealingWarmRestarts(1.0, 2, T_mult=2)
    assert abs(wr.step_to(2) - 1.0) < 1e-12 and abs(wr.step_to(6) - 1.0) < 1e-12
    w = S.WarmupThen(S.LinearWarmup(0.0, 1.0, 4), S.CosineAnnealingLR(1.0, 10))
    assert [round(w.step(), 4) for _ in range(5)] == [0.0, 0.25, 0.5, 0.75, 1.0]
    ch = S.ChainedLR([S.StepLR(1.0, 1, 0.5), S.ExponentialLR(0.1, 0.1)], [2, 2])
    assert [round(ch.step(), 6) for _ in range(4)] == [1.0, 0.5, 0.1, 0.01]
    sd = c.state_dict()
    assert sd.startswith("{'type':'CosineAnnealingLR'")
    c2 = S.CosineAnnealingLR(9.0, 3)
    assert c2.load_state_dict(sd) and c2.T_max == 10 and c2.last_epoch == 5
    r = S.ReduceLROnPlateau(1.0, factor=0.5, patience=1)
    lrs = [r.step(v) for v in [1.0, 1.0, 1.0, 1.0]]
    assert lrs == [1.0, 1.0, 0.5, 0.5]
    simple = L.CosineAnnealingLR(1.0, 4)
    assert [round(simple.step(), 4) for _ in range(5)] == [1.0, 0.8536, 0.5, 0.1464, 1.0]


def test_grad_scaler_state_machine():
    g = L.GradScaler(init_scale=1024.0, growth_interval=2)

    class Opt:
        steps = 0

        def step(self):
            self.steps += 1

        def zero_grad(self):
            pass

    o = Opt()
    assert g.step_and_update(o, found_inf=True) is False and o.steps == 0 and g.get_scale() == 512.0
    assert g.step_and_update(o, False) and g.step_and_update(o, False)
    assert o.steps == 2 and g.get_scale() == 1024.0
    assert g.check_overflow([torch.tensor([1.0, float("inf")])]) is True
    assert g.check_overflow([torch.ones(3)]) is False
    assert L.GradScaler(enabled=False).scale(3.0) == 3.0


def test_optimizers_match_torch():
    torch.manual_seed(0)
    w0 = torch.randn(5, 3)
    g = torch.randn(5, 3)
    for ours, ref in [
        (lambda p: L.SGD([p], lr=0.1, momentum=0.9), lambda p: torch.optim.SGD([p], lr=0.1, momentum=0.9)),
        (lambda p: L.AdamW([p], lr=0.01, weight_decay=0.1), lambda p: torch.optim.AdamW([p], lr=0.01, weight_decay=0.1)),
        (lambda p: L.Adagrad([p], lr=0.1), lambda p: torch.optim.Adagrad([p], lr=0.1)),
    ]:
        a, b = torch.nn.Parameter(w0.clone()), torch.nn.Parameter(w0.clone())
        oa, ob = ours(a), ref(b)
        for _ in range(4):
            a.grad, b.grad = g.clone(), g.clone()
            oa.step()
            ob.step()
        assert torch.allclose(a, b, atol=1e-5), type(oa).__name__
    lin = L.Linear(3, 2, dtype=torch.float32)
    before = lin.weight.detach().clone()
    L.SGD(0.5).step_linear(lin, torch.ones(2, 3), torch.ones(2))
    assert torch.allclose(lin.weight, before - 0.5)


def test_mnp_layout_a_roundtrip_and_reference_header(tmp_path):
    net = L.Sequential(L.Linear(4, 3, dtype=torch.float32), L.ReLU(), L.Linear(3, 2, dtype=torch.float32))
    base = str(tmp_path / "ckpt.mnp")
    L.utils.save_state_dict(net, base, extra={"step": 7})
    header = open(base + ".json").read()
    assert header.startswith('{"format":"MNP","version":1,"created_at":"1970-01-01T00:00:00Z","model_class":"Model","files":{"state":"')
    assert L.utils.read_model_class_from_header(base) == "Model" and L.utils.exists_checkpoint(base)
    state = json.loads(open(base + ".state.json").read())
    assert state["type"] == "Sequential" and state["num_modules"] == 3
    assert state["children"][0]["weight"] == "tensor(dtype=Float32, shape=[3, 4])"
    net2 = L.Sequential(L.Linear(4, 3, dtype=torch.float32), L.ReLU(), L.Linear(3, 2, dtype=torch.float32))
    assert L.utils.load_state_dict(net2, base)
    assert torch.equal(net2.get(2).weight, net.get(2).weight)
    assert L.utils.checkpoint.read_extra(base)["step"] == 7
    # a reference-written checkpoint (no blob, total_elems 0) still loads
    ref_base = str(tmp_path / "ref.mnp")
    open(ref_base + ".json", "w").write(
        '{"format":"MNP","version":1,"created_at":"1970-01-01T00:00:00Z","model_class":"Model","files":{"state":"'
        + ref_base + '.state.json","blob":"' + ref_base + '.bin"},"blob_meta":{"dtype":"float32","endian":"little","total_elems":0}}')
    open(ref_base + ".state.json", "w").write(net.state_json())
    assert L.utils.load_state_dict(net2, ref_base)
    assert not L.utils.load_state_dict(net2, str(tmp_path / "missing"))


def test_mnp_layout_b_and_csv_blob(tmp_path):
    net = L.Sequential(L.Linear(2, 2, dtype=torch.float32), L.Conv2d(1, 2, 3, dtype=torch.float32))
    header, flat = L.make_checkpoint(net)
    assert header == '{"params":[{"type":"Linear","w":4,"b":2},{"type":"Conv2d","w":18,"b":2}]}'
    assert flat.numel() == 26
    hp, bp = str(tmp_path / "n.header.json"), str(tmp_path / "n.state.bin")
    assert L.save_checkpoint_files(net, hp, bp)
    blob_text = open(bp).read()
    assert blob_text.count(",") == 25 and all(c in "0123456789.,-e+" for c in blob_text)
    ok, h2, b2 = L.load_checkpoint_files(hp, bp)
    assert ok and h2 == header and torch.allclose(b2, flat, atol=1e-7)
    net2 = L.Sequential(L.Linear(2, 2, dtype=torch.float32), L.Conv2d(1, 2, 3, dtype=torch.float32))
    assert L.apply_checkpoint(net2, h2, b2) and torch.allclose(net2.get(1).weight, net.get(1).weight, atol=1e-7)
    assert L.unpack_f64(L.pack_f64(torch.tensor([1.0, -2.5]))).tolist() == [1.0, -2.5]


def test_model_checkpoint_callback_names(tmp_path):
    net = L.Sequential(L.Linear(2, 2, dtype=torch.float32))
    mc = L.ModelCheckpoint(str(tmp_path), "run")
    mc.set_monitor("val_loss")
    mc.update_metric(0.5)
    mc.save(net, 3)
    names = set(os.listdir(tmp_path))
    assert {"run_step=3.mnp.json", "last.mnp.json", "best_val_loss.mnp.json"} <= names


def test_streaming_metric_merge_matches_single_pass():
    xs = [float(i * i % 7) for i in range(40)]
    a, b, full = L.metrics.StreamingMetric(), L.metrics.StreamingMetric(), L.metrics.StreamingMetric()
    a.update_many(xs[:13])
    b.update_many(xs[13:])
    full.update_many(xs)
    a.merge(b)
    assert a.count() == full.count() and abs(a.mean() - full.mean()) < 1e-12 and abs(a.variance() - full.variance()) < 1e-9
    assert (a.min(), a.max()) == (full.min(), full.max()) and abs(a.sum() - sum(xs)) < 1e-9
    cm = L.metrics.ConfusionMatrixBinary()
    assert cm.update_batch_scores([0.9, 0.2, 0.7, 0.1], [1, 0, 0, 1]) == 4
    assert (cm.tp(), cm.fp(), cm.tn(), cm.fn()) == (1, 1, 1, 1) and cm.balanced_accuracy() == 0.5 and cm.compute() == 0.5
    w = L.metrics.WeightedStreamingMetric()
    assert w.update_batch([1.0, 3.0, 9.0], [1.0, 1.0, 0.0]) == 3 and w.mean() == 2.0 and w.max() == 3.0 and w.weight_sum() == 2.0


def test_early_stopping_and_hooks_order():
    es = L.EarlyStopping(patience=2, mode="min")
    stops = [es.on_epoch_end(i, v) for i, v in enumerate([1.0, 0.9, 0.95, 0.97])]
    assert stops == [False, False, False, True] and es.get_best() == (0.9, 1)
    events = []

    class CB:
        def on_fit_start(self): events.append("fit_start")
        def on_epoch_start(self, e): events.append(f"epoch_start{e}")
        def on_batch_start(self, s): events.append(f"b{s}")
        def on_batch_end(self, s, msg): events.append(f"e{s}:{msg[:5]}")
        def on_epoch_end(self, e, status): events.append(f"epoch_end{e}:{status}")

    X, Y = torch.randn(8, 4), torch.randint(0, 2, (8,))
    net = L.Sequential(L.Linear(4, 2, dtype=torch.float32))
    steps = []

    class Opt(L.SGD):
        def step(self):
            steps.append(1)
            super().step()

    tr = L.Trainer(epochs=1, grad_accum_steps=2, verbose=False)
    tr.set_optimizer(Opt(net.parameters(), lr=0.1)).set_loss(torch.nn.functional.cross_entropy).set_callbacks([CB()])
    tr.fit(net, L.DataLoader(L.TensorDataset(X, Y), batch_size=2, shuffle=False))
    assert events[0] == "fit_start" and events[1] == "epoch_start0" and events[-1] == "epoch_end0:OK"
    assert events[2:4] == ["b0", "e0:loss="] and len(steps) == 2     # 4 batches / accumulate 2


def test_dropout_same_mask_every_call_and_layers():
    d = L.Dropout(0.5, seed=99)
    x = torch.ones(1000)
    assert torch.equal(d(x, True), d(x, True)) and 0.3 < (d(x, True) == 0).float().mean() < 0.7
    assert torch.equal(d(x, False), x)
    mp = L.MaxPool2d(2)
    assert mp(torch.randn(1, 1, 5, 5)).shape == (1, 1, 4, 4)      # default stride 1
    ct = L.ConvTranspose2d(2, 3, 3, (2, 2), (1, 1), dtype=torch.float32)
    assert ct(torch.randn(1, 2, 4, 4)).shape[-1] == (4 - 1) * 2 - 2 + 3
    ap = L.AvgPool2d(2, padding=(1, 1))
    assert torch.allclose(ap(torch.ones(1, 1, 4, 4)), torch.ones(1, 1, 3, 3))   # in-bounds average
    q = L.api.prepare(L.Sequential(L.Linear(4, 3, dtype=torch.float32)))
    xs = torch.randn(16, 4)
    ref = q.model(xs)
    q.calibrate([xs])
    cq = L.api.convert(q)
    assert (cq(xs) - ref).abs().max() < 0.05 * ref.abs().max() + 1e-3


def test_mha_softmax_and_relu_norm_match_manual():
    torch.manual_seed(0)
    m = L.MultiHeadAttention(8, 2, dtype=torch.float32)
    x = torch.randn(5, 1, 8)
    y = m(x)
    q, k, v = m.Wq(x[:, 0]), m.Wk(x[:, 0]), m.Wv(x[:, 0])
    outs = []
    for h in range(2):
        s = q[:, h * 4:(h + 1) * 4] @ k[:, h * 4:(h + 1) * 4].t() / 2.0
        outs.append(torch.softmax(s, -1) @ v[:, h * 4:(h + 1) * 4])
    assert torch.allclose(y[:, 0], m.Wo(torch.cat(outs, 1)), atol=1e-5)
    m.normalizer = "relu_norm"
    assert torch.isfinite(m(x)).all()
