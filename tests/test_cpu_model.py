"""The flagship model and the flat-buffer engine on CPU (plain torch path of every op)."""
import torch

from momijo_b200.models import GPT2, GPT2Config
from momijo_b200.parallel import ShardedDataParallel, AdamWConfig


def test_gpt2_cpu_trains():
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=200, n_layer=2, n_head=2, d_model=64, d_ff=128, max_seq=32,
                     dtype=torch.float32)
    model = GPT2(cfg)
    tok = torch.randint(0, cfg.vocab_size, (4, 17))
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    losses = []
    for _ in range(20):
        loss = model(tok[:, :-1], tok[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.7 * losses[0]
    lg = model.logits(tok[:, :-1])
    assert lg.shape == (4, 16, cfg.vocab_size)


def test_engine_cpu_flat_step_matches_torch_adamw():
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=100, n_layer=1, n_head=2, d_model=32, d_ff=64, max_seq=16,
                     dtype=torch.float32)
    m1, m2 = GPT2(cfg), GPT2(cfg)
    m2.load_state_dict(m1.state_dict())
    eng = ShardedDataParallel(m1, AdamWConfig(lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1))
    # the CPU engine keeps fp32 views when the module is fp32
    opt = torch.optim.AdamW(m2.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    tok = torch.randint(0, cfg.vocab_size, (2, 9))
    for _ in range(3):
        l1 = eng(tok[:, :-1], tok[:, 1:])
        l1.backward()
        eng.step()
        l2 = m2(tok[:, :-1], tok[:, 1:])
        opt.zero_grad()
        l2.backward()
        opt.step()
    assert abs(l1.item() - l2.item()) < 5e-2
