"""End-to-end GPT-2 step on the native kernels vs the same model evaluated by plain torch."""
import pytest
import torch

from momijo_b200 import _C
from momijo_b200.models import GPT2, GPT2Config
from momijo_b200.parallel import ShardedDataParallel, AdamWConfig

pytestmark = pytest.mark.gpu


def test_gpt2_loss_and_grads_match_reference_path():
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=1000, n_layer=2, n_head=2, d_model=128, d_ff=512, max_seq=256)
    model = GPT2(cfg).cuda()
    ref = GPT2(cfg)
    ref.load_state_dict(model.state_dict())
    ref = ref.float()  # CPU fp32 path of every op
    tok = torch.randint(0, cfg.vocab_size, (2, 257), device="cuda")
    loss = model(tok[:, :-1], tok[:, 1:])
    loss.backward()
    tc = tok.cpu()
    ref.cfg.dtype = torch.float32
    lr = ref(tc[:, :-1], tc[:, 1:])
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-2 * abs(lr.item()), (loss.item(), lr.item())
    got = dict(model.named_parameters())
    for name, p in ref.named_parameters():
        g, r = got[name].grad.float().cpu(), p.grad
        err = (g - r).abs().max().item() / (r.abs().max().item() + 1e-8)
        assert err < 8e-2, f"{name}: {err}"


def test_engine_trains_and_counts_launches():
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    eng = ShardedDataParallel(GPT2(cfg).cuda(), AdamWConfig(lr=1e-3))
    tok = torch.randint(0, cfg.vocab_size, (4, 129), device="cuda")
    before = _C.launches
    losses = []
    for _ in range(8):
        loss = eng(tok[:, :-1], tok[:, 1:])
        loss.backward()
        eng.step()
        losses.append(loss.item())
    assert _C.launches - before > 8 * 20
    assert losses[-1] < losses[0]


def test_micro_batch_accumulation_in_fp32_matches_reference():
    """Four micro-batches of (loss / 4).backward() into an fp32 gradient buffer == the gradient of the mean loss
    over the four micro-batches from the fp32 reference path; then one optimizer step."""
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=1000, n_layer=2, n_head=2, d_model=128, d_ff=512, max_seq=256)
    model = GPT2(cfg).cuda()
    ref = GPT2(cfg)
    ref.load_state_dict(model.state_dict())
    ref = ref.float()
    ref.cfg.dtype = torch.float32
    eng = ShardedDataParallel(model, AdamWConfig(lr=1e-3), grad_dtype=torch.float32)
    assert eng.flat.grad.dtype == torch.float32
    tok = torch.randint(0, cfg.vocab_size, (8, 129), device="cuda")
    for m in range(4):
        t = tok[2 * m:2 * m + 2]
        (eng(t[:, :-1], t[:, 1:]) / 4).backward()
    tc = tok.cpu()
    ref(tc[:, :-1], tc[:, 1:]).backward()
    got = dict(model.named_parameters())
    num = den = 0.0
    for name, p in ref.named_parameters():
        g = got[name].main_grad.float().cpu()
        num += (g - p.grad).pow(2).sum().item()
        den += p.grad.pow(2).sum().item()
    assert (num / den) ** 0.5 < 2e-2, (num / den) ** 0.5
    before = model.wte.detach().float().clone()
    eng.step()
    assert (model.wte.detach().float() - before).abs().max().item() > 0
