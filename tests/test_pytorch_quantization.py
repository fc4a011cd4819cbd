"""Quantisation toolkit: quantisation functions against closed forms, calibrators on known distributions, the quantiser's
switches, quantised layers, module swapping, the calibrate -> fine-tune workflow."""
import math

import numpy as np
import pytest
import torch
import torch.nn as tnn

from oslo_b200.lightseq import pytorch_quantization as pq
from oslo_b200.lightseq.pytorch_quantization import nn as qnn
from oslo_b200.lightseq.pytorch_quantization.tensor_quant import tensor_quant


def test_quant_functions_match_closed_forms_and_pass_gradients_inside_the_range():
    x = torch.tensor([-3.0, -1.0, -0.26, 0.0, 0.249, 0.5, 1.0, 2.0], requires_grad=True)
    codes, scale = tensor_quant(x, torch.tensor(1.0), 8, False, True)
    assert float(scale) == 127.0
    assert codes.tolist() == [-127, -127, -33, 0, 32, 64, 127, 127]
    wide, _ = tensor_quant(x, torch.tensor(1.0), 8, False, False)
    assert wide[0] == -128  # full range keeps the most negative code
    y = pq.fake_tensor_quant(x, torch.tensor(1.0), 8, False, True)
    assert torch.allclose(y, codes / 127.0)
    y.sum().backward()
    assert x.grad.tolist() == [0, 1, 1, 1, 1, 1, 1, 0]
    # per-axis amax, zero amax rows quantise to zero, 4 bits
    w = torch.tensor([[0.5, -1.0], [0.0, 0.0], [7.0, 3.5]])
    q = pq.fake_tensor_quant(w, pq.reduce_amax(w, axis=0), 4, False, True)
    assert torch.allclose(q, torch.tensor([[4 / 7, -1.0], [0.0, 0.0], [7.0, 4.0]]), atol=1e-6) or torch.allclose(q[2], torch.tensor([7.0, 4.0]))
    assert q[1].tolist() == [0.0, 0.0]
    # unsigned: 0..255 codes
    u, s = tensor_quant(torch.tensor([0.0, 0.5, 1.0]), torch.tensor(1.0), 8, True, False)
    assert u.tolist() == [0, 128, 255] and float(s) == 255.0
    with pytest.raises(ValueError):
        tensor_quant(torch.tensor([-1.0]), torch.tensor(1.0), 8, True, False)
    # affine: grid of 255 steps over [0, 2.55]
    a = torch.tensor([-1.0, 0.0, 0.014, 1.0, 2.55, 9.0], requires_grad=True)
    f = pq.fake_affine_tensor_quant(a, 0.0, 2.55, 8)
    assert torch.allclose(f, torch.tensor([0.0, 0.0, 0.01, 1.0, 2.55, 2.55]), atol=1e-6)
    f.sum().backward()
    assert a.grad.tolist() == [0, 1, 1, 1, 1, 0]


def test_descriptor_round_trip_and_validation():
    d = pq.QuantDescriptor(num_bits=4, axis=0, calib_method="histogram", unsigned=True)
    assert pq.QuantDescriptor.from_yaml(d.to_yaml()) == d and d.dict() == {"num_bits": 4, "axis": 0, "calib_method": "histogram", "unsigned": True}
    assert pq.QuantDescriptor().dict() == {}
    for bad in (dict(num_bits=0), dict(calib_method="median"), dict(learn_amax=True), dict(amax="x")):
        with pytest.raises((ValueError, TypeError)):
            pq.QuantDescriptor(**bad)


def test_max_and_histogram_calibrators():
    torch.manual_seed(0)
    m = pq.MaxCalibrator(8, axis=0, track_amax=True)
    a, b = torch.randn(4, 16), 3 * torch.randn(4, 16)
    m.collect(a)
    m.collect(b)
    want = torch.maximum(a.abs().amax(1, keepdim=True), b.abs().amax(1, keepdim=True))
    assert torch.equal(m.compute_amax(), want) and len(m.amaxs) == 2
    with pytest.raises(RuntimeError):
        m.collect(torch.randn(5, 16))
    m.reset()
    assert m.compute_amax() is None

    h = pq.HistogramCalibrator(8, None, False, num_bins=1024)
    x = torch.randn(200_000)
    h.collect(x[:100_000])
    h.collect(4.0 * x[100_000:] / x[100_000:].abs().max() * 1.7 * x.abs().max())  # larger values: the range has to grow
    counts, edges = h.histogram
    assert counts.sum() == 200_000 and len(counts) > 1024 and abs(edges[1] - edges[0] - x[:100_000].abs().max().item() / 1024) < 1e-9
    g = pq.HistogramCalibrator(8, None, False, num_bins=2048)
    g.collect(x)
    p999 = g.compute_amax("percentile", percentile=99.9)
    assert abs(float(p999) - np.percentile(x.abs().numpy(), 99.9)) < 0.02
    full = float(x.abs().max())
    mse, ent = float(g.compute_amax("mse")), float(g.compute_amax("entropy", stride=4))
    assert 0.5 * full < mse <= full * 1.001  # 8 bits: clipping a Gaussian costs more than it saves
    assert 0.3 * full < ent <= full * 1.001
    # a heavy outlier: both adaptive methods clip it away, max keeps it
    y = torch.cat([torch.randn(50_000), torch.tensor([60.0])])
    o = pq.HistogramCalibrator(4, None, False, num_bins=4096)
    o.collect(y)
    assert float(o.compute_amax("mse", start_bin=16)) < 10 and float(o.compute_amax("percentile", percentile=99.9)) < 5
    with pytest.raises(TypeError):
        o.compute_amax("median")
    with pytest.raises(NotImplementedError):
        pq.HistogramCalibrator(8, axis=0)


def test_tensor_quantizer_switches_state_dict_and_learned_amax():
    torch.manual_seed(1)
    q = pq.TensorQuantizer(pq.QuantDescriptor(num_bits=8))
    x = torch.randn(8, 32)
    dyn = q(x)  # no amax: dynamic range of the input
    assert (dyn - x).abs().max() <= x.abs().max() / 127 / 2 + 1e-6
    q.disable_quant()
    q.enable_calib()
    assert torch.equal(q(x), x) and torch.equal(q(2 * x), 2 * x)
    q.load_calib_amax()
    assert torch.isclose(q.amax, (2 * x).abs().max())
    q.enable_quant()
    q.disable_calib()
    clipped = q(10 * x)
    assert clipped.abs().max() <= q.amax * 128 / 127 + 1e-6  # the full-range grid has one more negative code
    assert "amax=" in repr(q) and "[Q]" in repr(q)
    # a calibrated quantiser's state loads into a fresh one (which has no amax buffer yet), also per-axis shapes
    fresh = pq.TensorQuantizer(pq.QuantDescriptor(num_bits=8))
    fresh.load_state_dict(q.state_dict())
    assert torch.equal(fresh.amax, q.amax)
    row = pq.TensorQuantizer(pq.QuantDescriptor(axis=0))
    row.amax = torch.ones(8, 1)
    again = pq.TensorQuantizer(pq.QuantDescriptor(axis=0))
    again.load_state_dict(row.state_dict())
    assert again.amax.shape == (8, 1)
    with pytest.raises(RuntimeError):
        pq.TensorQuantizer().load_calib_amax()
    # learned amax: elements beyond the range push it outwards
    lq = pq.TensorQuantizer(pq.QuantDescriptor(amax=1.0, learn_amax=True))
    out = lq(torch.tensor([0.2, 3.0, -5.0]))
    out.sum().backward()
    assert isinstance(lq.amax, tnn.Parameter) and lq.amax.grad is not None and float(lq.amax.grad) == 0.0  # +1 and -1 cancel
    lq.amax.grad = None
    lq(torch.tensor([0.2, 3.0, 5.0])).sum().backward()
    assert float(lq.amax.grad) == 2.0
    # clip stage: clamps without rounding
    cq = pq.TensorQuantizer(pq.QuantDescriptor(amax=1.0), if_quant=False, if_clip=True)
    assert cq(torch.tensor([0.3337, 2.0])).tolist() == [pytest.approx(0.3337), 1.0]
    # real (integer) mode exposes the scale
    rq = pq.TensorQuantizer(pq.QuantDescriptor(fake_quant=False, amax=2.0, narrow_range=True))
    codes = rq(torch.tensor([1.0, -2.0]))
    assert codes.tolist() == [64.0, -127.0] and float(rq.scale) == 63.5


def test_quantised_layers_track_their_float_versions():
    torch.manual_seed(2)
    x = torch.randn(2, 3, 12, 12)
    for qcls, fcls, args in ((pq.QuantConv2d, tnn.Conv2d, (3, 5, 3)), (qnn.QuantConvTranspose2d, tnn.ConvTranspose2d, (3, 5, 3))):
        ql = qcls(*args)
        fl = fcls(*args)
        fl.load_state_dict({k: v for k, v in ql.state_dict().items() if "quantizer" not in k})
        err = (ql(x) - fl(x)).abs().max() / fl(x).abs().max()
        assert 0 < err < 0.05, (qcls.__name__, float(err))
        assert ql.weight_quantizer.axis == (1 if "Transpose" in qcls.__name__ else 0)
    lin = pq.QuantLinear(32, 16, quant_desc_input=pq.QuantDescriptor(num_bits=4))
    assert lin.input_quantizer.num_bits == 4 and lin.weight_quantizer.axis == 0
    with pytest.raises(TypeError):
        pq.QuantLinear(4, 4, quant_desc_wieght=None)
    pool = qnn.QuantAvgPool2d(2)
    assert pool(x).shape == (2, 3, 6, 6) and isinstance(pool.input_quantizer, pq.TensorQuantizer)
    emb = pq.QuantEmbedding(50, 8, padding_idx=0)
    ids = torch.tensor([[1, 2, 0]])
    assert (emb(ids) - tnn.functional.embedding(ids, emb.weight)).abs().max() < emb.weight.abs().max() / 100
    att = pq.QuantSelfAttention(32, 4)
    h = torch.randn(2, 6, 32, requires_grad=True)
    att(h).sum().backward()
    assert h.grad is not None and sum(1 for _ in att.modules() if isinstance(_, pq.TensorQuantizer)) == 12


class _Net(tnn.Module):
    def __init__(self):
        super().__init__()
        self.body = tnn.Sequential(tnn.Linear(16, 32), tnn.ReLU(), tnn.Linear(32, 32), tnn.ReLU())
        self.head = tnn.Linear(32, 4)

    def forward(self, x):
        return self.head(self.body(x))


def test_module_swapping_global_and_in_place():
    plain = type(tnn.Linear(2, 2))
    with pq.quantized_construction(float_module_list=["Conv1d"]):
        net = _Net()
        assert isinstance(net.head, pq.QuantLinear) and type(tnn.Conv1d(1, 1, 1)).__name__ == "Conv1d"
        with pytest.raises(RuntimeError):
            pq.initialize()
    assert tnn.Linear is plain and type(_Net().head) is plain
    net = _Net()
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    ids = [id(p) for p in net.parameters()]
    n = pq.replace_with_quant(net, skip=["head"])
    assert n == 2 and isinstance(net.body[0], pq.QuantLinear) and type(net.head) is plain
    assert [id(p) for p in net.parameters()] == ids and opt.param_groups[0]["params"][0] is net.body[0].weight


def test_calibrate_then_finetune_workflow_and_optim_helpers():
    torch.manual_seed(3)
    net = _Net()
    data = [torch.randn(64, 16) for _ in range(6)]
    target = [net(x).detach() for x in data]
    pq.replace_with_quant(net, quant_desc_input=pq.QuantDescriptor(num_bits=4, calib_method="histogram"),
                          quant_desc_weight=pq.QuantDescriptor(num_bits=4, axis=0))
    assert pq.collect_stats(net, data, num_batches=4) == 4
    pq.compute_amax(net, "percentile", percentile=99.9)
    assert all(q.amax is not None for q in net.modules() if isinstance(q, pq.TensorQuantizer))
    pq.qat_mode(net)
    loss_fn = lambda: sum(((net(x) - t) ** 2).mean() for x, t in zip(data, target)) / len(data)
    before = float(loss_fn().detach())
    groups = pq.group_parameters(net, [[r"body\..*weight"], [r"head\."]], lrs=[3e-4, 2e-4])
    assert len(groups[0]["params"]) == 2 and len(groups[1]["params"]) == 2
    with pytest.raises(ValueError):
        pq.group_parameters(net, [[r"body"], [r"body\.0"]])
    assert pq.freeze_parameters(net, [r".*bias"]) == 3
    opt = torch.optim.Adam(groups)
    for _ in range(100):
        opt.zero_grad()
        loss = loss_fn()
        loss.backward()
        opt.step()
    after = float(loss_fn().detach())
    assert after < 0.9 * before, (before, after)  # training through the straight-through estimator recovers accuracy
    # weights rounded in place: the output does not change, the weight quantisers are off
    pq.ptq_mode(net)
    ref = net(data[0]).detach()
    assert pq.quant_weight_inplace(net) == 3
    assert torch.allclose(net(data[0]), ref, atol=1e-5)
    levels = torch.unique(net.body[0].weight[0] / net.body[0].weight[0].abs().max() * 7).numel()
    assert levels <= 15
    # weight-only calibration by histogram per channel
    other = _Net()
    pq.replace_with_quant(other)
    pq.calibrate_weights(other, "percentile", percentile=99.0)
    wq = other.body[0].weight_quantizer
    assert wq.amax.shape == (32, 1) and (wq.amax.flatten() <= other.body[0].weight.abs().amax(1) * 1.01).all()
