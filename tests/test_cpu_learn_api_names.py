"""Names and semantics of the smaller public helpers of the learn package (losses, init, KL, data, utils)."""
import math

import torch

import momijo_b200.learn as L
from momijo_b200.learn import losses, metrics
from momijo_b200.learn.data import (BatchIter, DataLoader, Dataset, LCG32, RNG32, clamp_index, collate_pairs_varlen,
                                    collate_varlen_by, make_enumerate, make_index_list, make_index_slice,
                                    make_random_index_partition, make_zip, shuffle_inplace)
from momijo_b200.learn.nn import activations, functional, init, pool, regularizers
from momijo_b200.learn.prob import kl_losses as K
from momijo_b200.learn.prob.distributions import Bernoulli, Normal
from momijo_b200.learn.utils import fileio_stub, profiling, randomness


def test_simple_lcg_matches_the_reference_recurrence():
    r = init.SimpleLCG()
    s = (6364136223846793005 * 88172645463393265 + 1) % (1 << 64)
    assert r.rand01() == (s >> 11) / 2.0 ** 53
    r2 = init.SimpleLCG(7)
    vals = [r2.rand01() for _ in range(12)]
    r3 = init.SimpleLCG(7)
    assert abs(r3.normal01() - (sum(vals) - 6.0)) < 1e-12


def test_init_bounds_and_fills():
    assert init.compute_fan_in_out([]) == (1, 1)
    assert init.compute_fan_in_out([5]) == (5, 5)
    assert init.compute_fan_in_out([8, 4, 3, 3]) == (36, 72)
    lo, hi = init.kaiming_uniform_bounds([8, 4], 0.0, "fan_in", "relu")
    assert abs(hi - math.sqrt(3.0) * math.sqrt(2.0) / 2.0) < 1e-12 and lo == -hi
    assert abs(init.xavier_normal_std([8, 4]) - math.sqrt(2.0 / 12)) < 1e-12
    arr = init.xavier_uniform_fill([0.0] * 6, [2, 3])
    t = torch.zeros(2, 3, dtype=torch.float64)
    init.xavier_uniform_fill_tensor(t)
    assert torch.allclose(t.reshape(-1), torch.tensor(arr, dtype=torch.float64))
    assert init.calculate_gain("unknown") == 1.0 and init.calculate_gain("selu") == 0.75


def test_losses_with_reference_names():
    x = torch.tensor([0.3, -1.2, 2.0], dtype=torch.float64)
    y = torch.tensor([1.0, 0.0, 1.0], dtype=torch.float64)
    p = torch.sigmoid(x)
    ce = torch.nn.functional.binary_cross_entropy_with_logits(x, y, reduction="none")
    ref = (torch.where(y == 1, 0.25, 0.75) * (1 - torch.where(y == 1, p, 1 - p)) ** 2 * ce).mean()
    assert abs(losses.focal_loss_binary_with_logits(x.tolist(), y.tolist()) - float(ref)) < 1e-12
    lg = [[1.0, 2.0, 0.5], [0.1, 0.2, 3.0]]
    a = losses.focal_loss_multiclass_with_logits(lg, [1, 2])
    b = losses.focal_loss_multiclass_with_logits(lg, [[0, 1, 0], [0, 0, 1]])
    assert abs(a - b) < 1e-12 and a > 0
    assert abs(losses.hinge_loss([0.5, -0.2, 2.0], [1, 0, 1]) - (0.5 + 0.8 + 0.0) / 3) < 1e-12
    assert losses.triplet_loss_from_dist([1.0, 2.0], [0.5, 5.0], 1.0, "sum") == 1.5
    assert losses.ranking.triplet_loss([[0.0, 0.0]], [[1.0, 0.0]], [[3.0, 4.0]], 1.0) == 0.0
    an = torch.ones(2, 2)
    assert float(losses.triplet_loss(an, an, an + 1.0, margin=5.0)) == 1.0     # 0 - 4 + 5
    assert float(losses.cosine_embedding_loss(an, an * 3, torch.tensor([1.0, -1.0]))) == 0.5
    assert abs(losses.dice_loss_mc([[1.0, 0.0]], [[1.0, 0.0]])) < 1e-6
    assert len(losses.iou_loss_mc_vec([[0.9, 0.1], [0.2, 0.8]], [[1, 0], [0, 1]])) == 2


def test_kl_functions():
    assert K.kl_normal_normal_scalar(0, 0, 1, 0) == 0.5
    assert K.kl_divergence(Normal(0, 1), Normal(1, 1)) == 0.5
    assert abs(K.kl_divergence(Bernoulli(0.3), Bernoulli(0.5)) - K.kl_bernoulli_scalar(0.3, 0.5)) < 1e-15
    assert K.kl_divergence_any(1, 2) == 0.0
    p, q = torch.rand(3, 4), torch.rand(3, 4)
    assert abs(float(K.kl_bernoulli_batched(p, q).sum()) - K.kl_bernoulli_sum(p, q)) < 1e-5
    assert K.kl_normal_normal_diag_batched(p, q, q, p).shape == (3,)
    assert abs(K.kl_categorical([0.2, 0.8], [0.5, 0.5]) - (0.2 * math.log(0.4) + 0.8 * math.log(1.6))) < 1e-12
    assert abs(K.kl_normal_normal_diag([0, 0], [0, 0], [1, 1], [0, 0]) - 1.0) < 1e-12


def test_metrics_activations_functional():
    assert metrics.argmax_index([1, 5, 5, 2]) == 1
    assert metrics.confusion_matrix_from_labels([0, 1, 1, 2, 9], [0, 1, 2, 2, 0], 3) == [[1, 0, 0], [0, 1, 0], [0, 1, 1]]
    assert metrics.f1_score_binary([0.9, 0.2, 0.7, 0.4], [1, 0, 0, 1]) == 0.5
    assert activations.hardsigmoid([0.0, 10.0]) == [0.5, 1.0]
    x = torch.arange(2 * 3 * 4 * 4, dtype=torch.float32).reshape(2, 3, 4, 4)
    idx = functional.im2col_indices(x, 3, 3, 1, 1)
    assert idx.shape == (2, 27, 16) and int(idx[0, 4, 5]) == 5    # centre tap of output (1, 1) is input (1, 1)
    back = functional.col2im_indices(torch.ones(idx.shape), idx, [2, 3, 4, 4])
    assert float(back[0, 0, 1, 1]) == 9.0 and float(back[0, 0, 0, 0]) == 0.0   # index 0 doubles as "padding"
    assert functional.conv2d_depthwise(x, torch.ones(3, 3, 3), 1, 1).shape == (2, 3, 4, 4)
    assert functional.conv2d_pointwise(x, torch.ones(5, 3)).shape == (2, 5, 4, 4)
    assert pool.pool2d_core(torch.arange(16.0).reshape(1, 1, 4, 4), 2).flatten().tolist() == [5.0, 7.0, 13.0, 15.0]
    w = torch.tensor([1.0, -2.0, 3.0])
    assert abs(regularizers.l2_penalty_tensor_f64(w, 0.1) - 0.7) < 1e-12
    assert abs(regularizers.elastic_net_penalty_tensors_f32([w, w], 0.1, 0.2, False) - 6.8) < 1e-5


def test_data_helpers():
    rng = LCG32(1)
    assert rng.next_u32() == (1664525 + 1013904223) % (1 << 32)
    idx = shuffle_inplace(list(range(8)), 1)
    assert sorted(idx) == list(range(8)) and idx != list(range(8))
    tr, va = make_random_index_partition(10, 0.7, 3)
    assert len(tr) == 7 and sorted(tr + va) == list(range(10))
    assert clamp_index(9, 4) == 3 and clamp_index(-2, 4) == 0 and clamp_index(1, 0) == 0
    assert make_zip([1, 2, 3], [4, 5, 6])[1] == (2, 5) and make_enumerate(["a", "b"])[1] == (1, "b")
    assert make_index_slice(list(range(10)), 2, 3)[2] == 4 and make_index_list([5, 6, 7], [2, 0])[0] == 7
    dl = DataLoader(Dataset(list(range(10))), batch_size=4, shuffle=True, drop_last=True, seed=7)
    assert list(BatchIter(dl)) == list(dl) and len(list(dl)) == 2
    it = dl._make_index_iter()
    assert it.remaining() == 10 and len(dl.next_batch(it)) == 4
    assert 1 <= RNG32(5).randint(1, 6) <= 6
    xb, yb = collate_pairs_varlen([([1, 2, 3], 0), ([4], 1)])
    assert xb.tolist() == [[1, 2, 3], [4, 0, 0]] and yb.tolist() == [0, 1]
    xb2, _ = collate_varlen_by([{"s": [7], "l": 2}], lambda d: d["s"], lambda d: d["l"])
    assert xb2.tolist() == [[7]]


def test_utils(tmp_path):
    assert profiling.ns_to_ms(2_500_000) == 2.5 and profiling.s_to_ns(-1) == 0 and profiling.s_to_ns(1.5) == 1_500_000_000
    f = str(tmp_path / "a.bin")
    assert fileio_stub.write_all_bytes(f, torch.tensor([1, 2, 255], dtype=torch.uint8))
    assert fileio_stub.read_all_bytes(f).tolist() == [1, 2, 255]
    assert fileio_stub.read_all_bytes(str(tmp_path / "missing")).numel() == 0
    assert randomness.randint(3, 0, 10) == randomness.randint(3, 0, 10)
    assert sorted(randomness.permutation(1, 5)) == [0, 1, 2, 3, 4]
    assert L.utils.checkpoint.exists_checkpoint_at(str(tmp_path), "none") is False


def test_kl_div_follows_the_reference_and_offers_the_log_input_form():
    import torch.nn.functional as F
    from momijo_b200.learn.losses import kl_div

    torch.manual_seed(0)
    p, q = torch.softmax(torch.randn(4, 5), -1), torch.softmax(torch.randn(4, 5), -1)
    want = float((p * (p / q).log()).sum())          # sum p log(p / q): losses.mojo:172-177
    assert abs(float(kl_div(p, q)) - want) < 1e-6
    assert float(kl_div(p, p)) == 0.0
    lp = torch.log_softmax(torch.randn(4, 5), -1)
    assert abs(float(kl_div(lp, q, log_input=True, reduction="batchmean")) -
               float(F.kl_div(lp, q, reduction="batchmean"))) < 1e-6
