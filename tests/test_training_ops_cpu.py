"""The training leftovers (loss, its gradient, AdamW, RMSProp) against PyTorch's own implementations."""
import pytest
import torch

from tensorsharp_b200.ops import training as T


def test_cross_entropy_matches_torch_with_label_smoothing():
    torch.manual_seed(0)
    logits = torch.randn(7, 11, requires_grad=True)
    tgt = torch.randint(0, 11, (7,))
    for ls in (0.0, 0.1):
        want = torch.nn.functional.cross_entropy(logits, tgt, label_smoothing=ls)
        probs = torch.softmax(logits.detach(), -1)
        assert abs(T.cross_entropy_loss(probs, tgt, label_smooth=ls) - float(want.detach())) < 1e-5
        (g,) = torch.autograd.grad(want, logits)
        got = T.cross_entropy_loss_backward(probs, tgt, label_smooth=ls)
        assert torch.allclose(got, g, atol=1e-6)
        acc = torch.ones(7, 11)
        T.cross_entropy_loss_backward(probs, tgt, label_smooth=ls, grad=acc, add_grad=True)
        assert torch.allclose(acc, g + 1, atol=1e-6)
    with pytest.raises(ValueError):
        T.cross_entropy_loss(torch.softmax(logits.detach(), -1), tgt, label_smooth=1.5)
    with pytest.raises(ValueError):
        T.smoothed_labels(torch.tensor([11]), 11)


def test_adam_step_matches_torch_adamw_and_zeroes_the_gradient():
    torch.manual_seed(1)
    w0 = torch.randn(5, 3)
    ref_w = w0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_w], lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05)
    w, m, v = w0.clone(), torch.zeros(5, 3), torch.zeros(5, 3)
    for it in range(1, 6):
        g = torch.randn(5, 3) * 0.5
        ref_w.grad = g.clone()
        opt.step()
        grad = g.clone()
        T.adam_step(w, grad, v, m, step_size=0.01, clip_value=100.0, regc=0.05, iteration=it)
        assert float(grad.abs().sum()) == 0.0
        assert torch.allclose(w, ref_w.detach(), atol=1e-5)
    big = torch.full((5, 3), 50.0)
    w1 = w.clone()
    T.adam_step(w1, big.clone(), v.clone(), m.clone(), step_size=0.01, clip_value=1.0, iteration=6)
    w2 = w.clone()
    T.adam_step(w2, torch.ones(5, 3), v.clone(), m.clone(), step_size=0.01, clip_value=1.0, iteration=6)
    assert torch.allclose(w1, w2)                       # gradients are clamped before the moments see them


def test_rmsprop_step_moves_against_the_gradient():
    w, g, c = torch.zeros(4), torch.tensor([1.0, -1.0, 0.5, 0.0]), torch.zeros(4)
    T.rmsprop_step(w, g, c, step_size=0.1, decay_rate=0.9)
    assert w[0] < 0 < w[1] and w[3] == 0 and float(g.abs().sum()) == 0.0
