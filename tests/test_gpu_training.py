"""A small training loop through the operator: a checkpointed block with low-rank adapters, five AdamW steps
under autocast, eager strict API and compiled automatic API against PyTorch's native attention (the caller
pattern the reference pins in tests/test_training.py:99-133 of the reference project)."""

import copy

import pytest
import torch
from torch.utils.checkpoint import checkpoint

pytestmark = pytest.mark.gpu


class AdapterLinear(torch.nn.Module):
    """A frozen projection plus a trainable rank-4 update that starts at zero."""

    def __init__(self, width, rank=4):
        super().__init__()
        self.frozen = torch.nn.Linear(width, width).requires_grad_(False)
        self.down = torch.nn.Linear(width, rank, bias=False)
        self.up = torch.nn.Linear(rank, width, bias=False)
        torch.nn.init.zeros_(self.up.weight)

    def forward(self, x):
        return self.frozen(x) + self.up(self.down(x))


class Block(torch.nn.Module):
    def __init__(self, attention, width=128, heads=2):
        super().__init__()
        self.attention, self.heads = attention, heads
        self.q, self.k, self.v, self.o = (AdapterLinear(width) for _ in range(4))

    def forward(self, x):
        split = lambda t: t.reshape(x.shape[0], x.shape[1], self.heads, -1).transpose(1, 2)  # BSHD projection views
        out = self.attention(split(self.q(x)), split(self.k(x)), split(self.v(x)))
        return x + self.o(out.transpose(1, 2).reshape(x.shape))


def test_checkpointed_adapter_training_matches_native_attention():
    import kohakufa_cute

    torch.manual_seed(99)
    native_sdpa = torch.nn.functional.scaled_dot_product_attention
    initial = Block(native_sdpa).cuda()
    x = torch.randn(1, 33, 128, device="cuda")
    target = torch.randn_like(x)
    histories, changes = [], []
    for fn, compiled in ((native_sdpa, False), (kohakufa_cute.scaled_dot_product_attention, False),
                         (kohakufa_cute.automatic_scaled_dot_product_attention, True)):
        model = copy.deepcopy(initial)
        model.attention = fn
        params = [p for p in model.parameters() if p.requires_grad]
        start = [p.detach().clone() for p in params]
        step_fn = torch.compile(model, fullgraph=True) if compiled else model
        optimizer = torch.optim.AdamW(params, lr=1e-3)
        history = []
        for _ in range(5):
            optimizer.zero_grad(set_to_none=True)
            inputs = x.detach().requires_grad_()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                output = checkpoint(step_fn, inputs, use_reentrant=False)
                loss = (output.float() - target).square().mean()
            loss.backward()
            assert all(p.grad is not None and bool(torch.isfinite(p.grad).all()) for p in params)
            optimizer.step()
            history.append(loss.detach())
        histories.append(torch.stack(history))
        changes.append(torch.cat([(p.detach() - s).flatten() for p, s in zip(params, start)]))
    for history, change in zip(histories[1:], changes[1:]):
        torch.testing.assert_close(history, histories[0], atol=1e-3, rtol=1e-2)
        assert float((change - changes[0]).norm()) < 0.05 * float(changes[0].norm())
        assert float(change.norm()) > 0
        assert float(history[-1]) < float(history[0])
