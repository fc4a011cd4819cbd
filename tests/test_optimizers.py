"""Optimizers on CPU tensors (pure-torch paths and the C++ host optimizers) against torch.optim references."""
import pytest
import torch


def _params(seed=0, dtype=torch.float32):
    torch.manual_seed(seed)
    return [torch.randn(s, dtype=dtype).requires_grad_() for s in [(33, 7), (5,), (130, 3)]]


def _run(opt_a, ps_a, opt_b, ps_b, steps=4):
    for s in range(steps):
        torch.manual_seed(50 + s)
        for a, b in zip(ps_a, ps_b):
            g = torch.randn_like(b)
            a.grad, b.grad = g.clone().to(a.dtype), g.clone()
        opt_a.step()
        opt_b.step()


def test_cpu_adam_matches_torch_adamw():
    from oslo_b200.optim import CPUAdam

    a, b = _params(), _params()
    _run(CPUAdam(a, lr=1e-2, weight_decay=0.1), a, torch.optim.AdamW(b, lr=1e-2, weight_decay=0.1), b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


def test_cpu_adam_l2_mode_and_lowp_copy():
    from oslo_b200.optim import CPUAdam

    a, b = _params(1), _params(1)
    copies = {p: torch.zeros_like(p, dtype=torch.bfloat16) for p in a}
    _run(CPUAdam(a, lr=1e-2, weight_decay=0.1, adamw_mode=False, param_copies=copies), a,
         torch.optim.Adam(b, lr=1e-2, weight_decay=0.1), b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)
        assert torch.equal(copies[x], x.detach().to(torch.bfloat16))


def test_cpu_adagrad_matches_torch():
    from oslo_b200.optim import CPUAdagrad

    a, b = _params(2), _params(2)
    _run(CPUAdagrad(a, lr=1e-2, weight_decay=0.01), a, torch.optim.Adagrad(b, lr=1e-2, weight_decay=0.01, eps=1e-10), b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


def test_fused_optimizers_torch_paths():
    from oslo_b200.optim import FusedAdagrad, FusedAdam, FusedLamb, FusedNovoGrad, FusedSGD

    a, b = _params(3), _params(3)
    _run(FusedAdam(a, lr=1e-2, weight_decay=0.1), a, torch.optim.AdamW(b, lr=1e-2, weight_decay=0.1), b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)
    a, b = _params(4), _params(4)
    _run(FusedSGD(a, lr=1e-2, momentum=0.9, weight_decay=0.01), a, torch.optim.SGD(b, lr=1e-2, momentum=0.9, weight_decay=0.01), b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)
    a, b = _params(5), _params(5)
    _run(FusedAdagrad(a, lr=1e-2), a, torch.optim.Adagrad(b, lr=1e-2, eps=1e-10), b)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)
    # LAMB / NovoGrad: finite, and the loss of a quadratic goes down
    for cls in (FusedLamb, FusedNovoGrad):
        torch.manual_seed(6)
        w = torch.randn(20, 20).requires_grad_()
        opt = cls([w], lr=5e-2)
        first = None
        for _ in range(30):
            opt.zero_grad()
            loss = (w ** 2).sum()
            loss.backward()
            opt.step()
            first = first or loss.item()
        assert torch.isfinite(w).all() and (w ** 2).sum().item() < first
