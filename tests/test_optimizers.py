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


def test_dynamic_loss_scaler_skips_overflow_and_adapts_the_scale():
    import torch

    from oslo_b200.optim import DynamicLossScaler

    w = torch.nn.Parameter(torch.ones(4))
    opt = torch.optim.SGD([w], lr=0.5)
    sc = DynamicLossScaler(init_scale=8.0, growth_interval=2)
    # clean step: the gradient is un-scaled exactly once, the step is taken
    sc.scale((w * torch.tensor([1.0, 2.0, 3.0, 4.0])).sum()).backward()
    assert w.grad.tolist() == [8.0, 16.0, 24.0, 32.0]
    assert sc.unscale_(opt) is False and sc.unscale_(opt) is False
    assert w.grad.tolist() == [1.0, 2.0, 3.0, 4.0]
    sc.step(opt)
    sc.update()
    assert w.tolist() == [0.5, 0.0, -0.5, -1.0] and sc.get_scale() == 8.0
    # overflow: no update, scale halves, counter resets
    opt.zero_grad()
    before = w.detach().clone()
    sc.scale((w * torch.tensor([1.0, float("inf"), 1.0, 1.0])).sum()).backward()
    assert sc.step(opt) is None
    sc.update()
    assert torch.equal(w.detach(), before) and sc.get_scale() == 4.0 and sc.skipped_steps == 1
    # two clean steps grow it again; the state round-trips
    for _ in range(2):
        opt.zero_grad()
        sc.scale(w.sum()).backward()
        sc.step(opt)
        sc.update()
    assert sc.get_scale() == 8.0
    other = DynamicLossScaler()
    other.load_state_dict(sc.state_dict())
    assert other.get_scale() == 8.0 and other.skipped_steps == 1 and other.growth_interval == 2
    off = DynamicLossScaler(enabled=False)
    assert off.get_scale() == 1.0 and off.scale(torch.tensor(3.0)).item() == 3.0
    with pytest.raises(ValueError):
        DynamicLossScaler(growth_factor=1.0)
