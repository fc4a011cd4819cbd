"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference (needs a B200)."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.fixture(autouse=True)
def _status():
    from oslo_b200.ops import _lib

    yield
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256])
def test_gemm_layouts(a_t, b_t, bn):
    from oslo_b200.ops.gemm import gemm

    torch.manual_seed(0)
    M, N, K = 392, 520, 200
    a = torch.randn((K, M) if a_t else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_t else (N, K), device=DEV, dtype=torch.bfloat16)
    A, B = (a.t() if a_t else a), (b.t() if b_t else b)
    y = gemm(A, B, block_n=bn)
    ref = A.float() @ B.float().t()
    assert _rel(y, ref) < 1e-2


def test_gemm_epilogues_and_batch():
    from oslo_b200.ops.gemm import gemm

    torch.manual_seed(1)
    a = torch.randn(512, 256, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(384, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float()
    assert _rel(gemm(a, b, bias=bias, epilogue="bias"), ref) < 1e-2
    aux = torch.empty(512, 384, device=DEV, dtype=torch.bfloat16)
    y = gemm(a, b, bias=bias, epilogue="gelu", aux=aux)
    assert _rel(y, F.gelu(ref, approximate="tanh")) < 1e-2
    assert _rel(aux, ref) < 1e-2
    c = torch.randn(512, 384, device=DEV, dtype=torch.bfloat16)
    c0 = c.float().clone()
    gemm(a, b, out=c, accumulate=True)
    assert _rel(c, c0 + a.float() @ b.float().t()) < 1e-2
    a4 = torch.randn(2, 3, 128, 64, device=DEV, dtype=torch.float16)
    b4 = torch.randn(2, 3, 256, 64, device=DEV, dtype=torch.float16)
    assert _rel(gemm(a4, b4), a4.float() @ b4.float().transpose(-1, -2)) < 1e-2


def test_linear_autograd():
    from oslo_b200.ops.gemm import linear

    torch.manual_seed(2)
    x = torch.randn(4, 96, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(256, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2
    assert _rel(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("h", [256, 2048, 4096, 5120])
@pytest.mark.parametrize("rms", [False, True])
def test_norm(dtype, h, rms):
    from oslo_b200.ops.norm import layer_norm, rms_norm, rms_norm_reference

    torch.manual_seed(3)
    x = torch.randn(37, 5, h, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(h, device=DEV) * 0.1 + 1).to(dtype).requires_grad_()
    b = (torch.randn(h, device=DEV) * 0.1).to(dtype).requires_grad_()
    g = torch.randn(37, 5, h, device=DEV, dtype=dtype)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    if rms:
        y = rms_norm(x, h, w, 1e-6)
        yr = rms_norm_reference(xr, wr, 1e-6)
    else:
        y = layer_norm(x, h, w, b, 1e-5)
        yr = F.layer_norm(xr, (h,), wr, br, 1e-5)
    y.backward(g)
    yr.backward(g.float())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert _rel(y, yr) < tol
    assert _rel(x.grad, xr.grad) < tol
    assert _rel(w.grad, wr.grad) < max(tol, 3e-2 if dtype != torch.float32 else tol)
    if not rms:
        assert _rel(b.grad, br.grad) < max(tol, 3e-2 if dtype != torch.float32 else tol)


def test_norm_mixed_dtype():
    from oslo_b200.ops.norm import layer_norm

    x = torch.randn(64, 1024, device=DEV, dtype=torch.bfloat16)
    w = torch.rand(1024, device=DEV) + 0.5
    b = torch.randn(1024, device=DEV)
    y = layer_norm(x, 1024, w, b, 1e-5)
    assert y.dtype == torch.bfloat16
    assert _rel(y, F.layer_norm(x.float(), (1024,), w, b, 1e-5)) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bias_gelu_swiglu_dropout(dtype):
    from oslo_b200.ops.activation import bias_dropout_add, bias_gelu, swiglu

    torch.manual_seed(4)
    x = torch.randn(33, 512, device=DEV, dtype=dtype, requires_grad=True)
    bias = torch.randn(512, device=DEV, dtype=dtype, requires_grad=True)
    g = torch.randn(33, 512, device=DEV, dtype=dtype)
    y = bias_gelu(x, bias)
    y.backward(g)
    xr, br = x.detach().float().requires_grad_(), bias.detach().float().requires_grad_()
    yr = F.gelu(xr + br, approximate="tanh")
    yr.backward(g.float())
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert _rel(y, yr) < tol and _rel(x.grad, xr.grad) < tol and _rel(bias.grad, br.grad) < 3e-2

    gu = torch.randn(17, 2 * 256, device=DEV, dtype=dtype, requires_grad=True)
    gg = torch.randn(17, 256, device=DEV, dtype=dtype)
    s = swiglu(gu)
    s.backward(gg)
    gur = gu.detach().float().requires_grad_()
    sr = F.silu(gur[:, :256]) * gur[:, 256:]
    sr.backward(gg.float())
    assert _rel(s, sr) < tol and _rel(gu.grad, gur.grad) < tol

    res = torch.randn(33, 512, device=DEV, dtype=dtype)
    out = bias_dropout_add(x.detach(), bias.detach(), res, 0.0, True)
    assert _rel(out, x.detach().float() + bias.detach().float() + res.float()) < tol
    xd = torch.ones(64, 4096, device=DEV, dtype=dtype, requires_grad=True)
    od = bias_dropout_add(xd, None, None, 0.25, True)
    kept = (od != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.02
    assert abs(od.float().mean().item() - 1.0) < 0.05
    od.sum().backward()
    assert torch.equal((xd.grad != 0), (od != 0))  # backward regenerates the same mask


@pytest.mark.parametrize("causal", [False, True])
def test_softmax(causal):
    from oslo_b200.ops.softmax import scale_mask_softmax, softmax_reference

    torch.manual_seed(5)
    x = torch.randn(2, 3, 64, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    mask = None if causal else (torch.rand(2, 1, 1, 64, device=DEV) > 0.8).float() * -10000.0
    y = scale_mask_softmax(x, 0.5, causal, mask)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = softmax_reference(xr, 0.5, causal, mask)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 2e-2


@pytest.mark.parametrize("neox", [True, False])
def test_rope(neox):
    from oslo_b200.ops.softmax import apply_rope, rope_reference, rope_tables

    torch.manual_seed(6)
    b, s, nh, hd, rot = 2, 32, 4, 64, 16
    qkv = torch.randn(b, s, nh, 3, hd, device=DEV, dtype=torch.bfloat16)
    cos, sin = rope_tables(s, rot, 10000.0, DEV)
    q_ref = rope_reference(qkv[..., 0, :].clone(), cos, sin, rot, neox)
    q = apply_rope(qkv[..., 0, :], cos, sin, rot, neox)  # in place on the strided view
    assert _rel(q, q_ref) < 1e-2
    back = apply_rope(q.clone().requires_grad_(), cos, sin, rot, neox)
    back.backward(torch.ones_like(back))


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("hd", [64, 128])
def test_flash_attention_backward(causal, hd):
    from oslo_b200.ops.attention import attention, attention_reference

    torch.manual_seed(17)
    b, s, nh = 2, 512, 2
    qkv = (torch.randn(b, s, nh, 3, hd, device=DEV) * 0.6).to(torch.bfloat16).requires_grad_()
    out = attention(qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :], causal=causal)
    g = torch.randn_like(out)
    out.backward(g)
    ref_in = qkv.detach().float().requires_grad_()
    ref = attention_reference(ref_in[..., 0, :], ref_in[..., 1, :], ref_in[..., 2, :], causal=causal)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    for i, name in enumerate("qkv"):
        assert _rel(qkv.grad[..., i, :], ref_in.grad[..., i, :]) < 4e-2, name


@pytest.mark.parametrize("causal", [True, False])
def test_attention(causal):
    from oslo_b200.ops.attention import attention, attention_reference

    torch.manual_seed(7)
    b, s, nh, hd = 2, 384, 4, 64
    qkv = (torch.randn(b, s, nh, 3, hd, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
    out = attention(q, k, v, causal=causal)
    g = torch.randn_like(out)
    out.backward(g)
    qkv_r = qkv.detach().float().requires_grad_()
    out_r = attention_reference(qkv_r[..., 0, :], qkv_r[..., 1, :], qkv_r[..., 2, :], causal=causal)
    out_r.backward(g.float())
    assert _rel(out, out_r) < 2e-2
    assert _rel(qkv.grad, qkv_r.grad) < 3e-2


def test_cross_entropy():
    from oslo_b200.ops.loss import vocab_parallel_cross_entropy

    torch.manual_seed(8)
    rows, v = 50, 1000
    logits = torch.randn(5, 10, v, device=DEV, dtype=torch.bfloat16)
    tgt = torch.randint(0, 990, (5, 10), device=DEV)
    tgt[0, :3] = -100
    lr = logits.detach().float().requires_grad_()
    lr_masked = lr.clone()
    lr_masked[..., 990:] = float("-inf")
    ref = F.cross_entropy(lr_masked.view(-1, v), tgt.view(-1), ignore_index=-100, reduction="none").view(5, 10)
    wts = torch.rand(5, 10, device=DEV) + 0.25  # a different upstream gradient per token: the backward scales row by row
    (ref * wts).sum().backward()
    x = logits.clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(x * 1.0, tgt, None, valid_vocab=990)
    (loss * wts).sum().backward()
    assert _rel(loss, ref) < 1e-3
    assert _rel(x.grad, lr.grad) < 2e-2


@pytest.mark.parametrize("dtype,master", [(torch.float32, False), (torch.bfloat16, True), (torch.float16, False)])
def test_fused_adam(dtype, master):
    from oslo_b200.optim import FusedAdam

    torch.manual_seed(9)
    shapes = [(300, 70), (17,), (4096, 33), (5,)]
    ps = [torch.randn(s, device=DEV, dtype=dtype).requires_grad_() for s in shapes]
    rs = [p.detach().float().clone().requires_grad_() for p in ps]
    opt = FusedAdam(ps, lr=1e-2, weight_decay=0.1, master_weights=master)
    ref = torch.optim.AdamW(rs, lr=1e-2, weight_decay=0.1)
    for _ in range(5):
        for p, r in zip(ps, rs):
            g = torch.randn_like(r)
            p.grad = g.to(dtype)
            r.grad = g.to(dtype).float()
        opt.step()
        ref.step()
    tol = 1e-5 if dtype == torch.float32 else (1e-2 if master else 3e-2)
    for p, r in zip(ps, rs):
        assert _rel(p, r) < tol
    if master:
        for p, r in zip(ps, rs):
            assert _rel(opt.state[p]["master"], r) < 1e-5


def test_neox_model_matches_reference_path():
    """Whole model on the native kernels vs the same weights on the pure-torch CPU path."""
    from oslo_b200.models.config import GPTNeoXConfig
    from oslo_b200.models.gpt_neox import GPTNeoXForCausalLM

    torch.manual_seed(10)
    cfg = GPTNeoXConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                        intermediate_size=512, max_position_embeddings=64)
    cpu = GPTNeoXForCausalLM(cfg)
    gpu = GPTNeoXForCausalLM(cfg)
    gpu.load_state_dict(cpu.state_dict())
    gpu = gpu.to(DEV, torch.bfloat16)
    ids = torch.randint(0, 512, (2, 64))
    l_cpu = cpu(input_ids=ids, labels=ids).loss
    l_gpu = gpu(input_ids=ids.to(DEV), labels=ids.to(DEV)).loss
    l_cpu.backward()
    l_gpu.backward()
    assert abs(l_cpu.item() - l_gpu.item()) < 3e-2
    gc = dict(cpu.named_parameters())
    for k, p in gpu.named_parameters():
        assert _rel(p.grad.cpu(), gc[k].grad) < 8e-2, k


@pytest.mark.parametrize("layout", ["h3d", "3hd"])
def test_qkv_attention_with_rope(layout):
    from oslo_b200.ops.attention import qkv_attention
    from oslo_b200.ops.softmax import rope_tables

    torch.manual_seed(11)
    b, s, nh, hd, rot = 2, 256, 4, 64, 16
    base = (torch.randn(b, s, 3 * nh * hd, device=DEV) * 0.5).to(torch.bfloat16)
    cos, sin = rope_tables(s, rot, 10000.0, DEV)
    x = base.clone().requires_grad_()
    out = qkv_attention(x * 1.0, nh, hd, layout=layout, causal=True, rope=(cos, sin, rot, True))
    g = torch.randn_like(out)
    out.backward(g)
    xr = base.float().cpu().requires_grad_()
    out_r = qkv_attention(xr * 1.0, nh, hd, layout=layout, causal=True, rope=(cos.cpu(), sin.cpu(), rot, True))
    out_r.backward(g.float().cpu())
    assert _rel(out.cpu(), out_r) < 2e-2
    assert _rel(x.grad.cpu(), xr.grad) < 3e-2


def test_moe_kernels_match_torch_paths():
    from oslo_b200.ops import moe

    torch.manual_seed(12)
    S, E, K, H, C = 300, 8, 2, 128, 96
    idx = torch.stack([torch.randint(0, E, (S,)), torch.randint(0, E, (S,))], 1).to(torch.int32)
    pos_g, cnt_g = moe.positions(idx.to(DEV), E)
    pos_c, cnt_c = moe.positions(idx, E)
    assert torch.equal(pos_g.cpu(), pos_c) and torch.equal(cnt_g.cpu(), cnt_c)
    slot = torch.where(pos_c < C, idx * C + pos_c, torch.full_like(pos_c, -1))
    x = torch.randn(S, H)
    w = torch.rand(S, K)
    xg = x.to(DEV, torch.bfloat16).requires_grad_()
    wg = w.to(DEV).requires_grad_()
    xr = x.to(torch.bfloat16).float().requires_grad_()
    wr = w.clone().requires_grad_()
    yg = moe.combine(moe.dispatch(xg, slot.to(DEV), E * C) * 1.5, wg, slot.to(DEV))
    yr = moe.combine(moe.dispatch(xr, slot, E * C) * 1.5, wr, slot)
    g = torch.randn(S, H)
    yg.backward(g.to(DEV, torch.bfloat16))
    yr.backward(g.to(torch.bfloat16).float())
    assert _rel(yg.cpu(), yr) < 2e-2
    assert _rel(xg.grad.cpu(), xr.grad) < 2e-2
    assert _rel(wg.grad.cpu(), wr.grad) < 3e-2


@pytest.mark.parametrize("name", ["sgd", "adagrad", "lamb", "novograd"])
def test_fused_optimizers_cuda_match_cpu_paths(name):
    from oslo_b200 import optim

    make = {"sgd": lambda ps: optim.FusedSGD(ps, lr=1e-2, momentum=0.9, weight_decay=0.01),
            "adagrad": lambda ps: optim.FusedAdagrad(ps, lr=1e-2, weight_decay=0.01),
            "lamb": lambda ps: optim.FusedLamb(ps, lr=1e-2, weight_decay=0.01),
            "novograd": lambda ps: optim.FusedNovoGrad(ps, lr=1e-2, weight_decay=0.01)}[name]
    torch.manual_seed(13)
    shapes = [(257, 33), (19,), (1024, 40)]
    cpu = [torch.randn(s).requires_grad_() for s in shapes]
    gpu = [p.detach().to(DEV).requires_grad_() for p in cpu]
    oc, og = make(cpu), make(gpu)
    for step in range(4):
        for a, b in zip(cpu, gpu):
            g = torch.randn_like(a)
            a.grad, b.grad = g, g.to(DEV)
        oc.step()
        og.step()
    for a, b in zip(cpu, gpu):
        assert _rel(b.cpu(), a) < 1e-4, name


def test_ngram_repeat_block_kernel():
    from oslo_b200.nn.ngram_repeat_block import NGramRepeatBlock, ngram_repeat_block_reference

    torch.manual_seed(14)
    rows, length, vocab, n = 12, 40, 50, 3
    tok = torch.randint(0, 6, (rows, length))
    lp = torch.randn(rows, vocab)
    ref = ngram_repeat_block_reference(tok, lp.clone(), 29, n)
    out = NGramRepeatBlock()(tok.to(DEV), lp.clone().to(DEV), rows, 29, 1, n)
    assert torch.equal(torch.isinf(out.cpu()), torch.isinf(ref))


def test_llama_and_gpt2_models_run_on_native_kernels():
    from oslo_b200.models import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM

    torch.manual_seed(15)
    ids = torch.randint(0, 512, (2, 64))
    for cls, cfg in [(LlamaForCausalLM, LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=352, num_hidden_layers=2,
                                                    num_attention_heads=4, max_position_embeddings=64)),
                     (GPT2LMHeadModel, GPT2Config(vocab_size=512, n_positions=64, n_embd=128, n_layer=2, n_head=4, resid_pdrop=0.0,
                                                  embd_pdrop=0.0, attn_pdrop=0.0))]:
        cpu = cls(cfg)
        gpu = cls(cfg)
        gpu.load_state_dict(cpu.state_dict())
        gpu = gpu.to(DEV, torch.bfloat16)
        lc = cpu(input_ids=ids, labels=ids).loss
        lg = gpu(input_ids=ids.to(DEV), labels=ids.to(DEV)).loss
        lc.backward()
        lg.backward()
        assert abs(lc.item() - lg.item()) < 5e-2, cls.__name__
        gc = dict(cpu.named_parameters())
        for k, p in gpu.named_parameters():
            assert _rel(p.grad.cpu(), gc[k].grad) < 0.1, (cls.__name__, k)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("hd", [64, 128])
def test_flash_attention_forward(causal, hd):
    from oslo_b200.ops.attention import attention_reference, flash_attention_forward

    torch.manual_seed(16)
    b, s, nh = 2, 512, 3
    qkv = (torch.randn(b, s, nh, 3, hd, device=DEV) * 0.7).to(torch.bfloat16)
    q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
    scale = 1.0 / math.sqrt(hd)
    out, lse = flash_attention_forward(q, k, v, causal, scale)
    ref = attention_reference(q.float(), k.float(), v.float(), causal=causal, scale=scale)
    assert _rel(out, ref) < 2e-2
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=DEV).tril(), float("-inf"))
    assert _rel(lse, torch.logsumexp(scores, dim=-1)) < 1e-3


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("hd,dtype", [(128, torch.bfloat16), (64, torch.bfloat16), (128, torch.float16)])
def test_flash_attention_forward_pingpong(causal, hd, dtype):
    """The one-pass forward (two query tiles per CTA, probabilities through tensor memory, lazy rescale of the output)
    against fp32: output and log-sum-exp, at a length with several key tiles per query block and scores large enough
    that the running maximum grows by more than the rescale threshold after the first tile."""
    from oslo_b200.ops.attention import attention_reference, flash_attention_forward

    torch.manual_seed(61)
    b, s, nh = 2, 1024, 3
    qkv = (torch.randn(b, s, nh, 3, hd, device=DEV) * 1.5).to(dtype)
    q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
    scale = 1.0 / math.sqrt(hd)
    out, lse = flash_attention_forward(q, k, v, causal, scale, pingpong=True)
    torch.cuda.synchronize()
    from oslo_b200.ops import _lib

    _lib.check_status()
    ref = attention_reference(q.float(), k.float(), v.float(), causal=causal, scale=scale)
    frac, worst = _close(out, ref, rtol=2e-2, atol=0.02)
    assert frac == 0.0, ("out", frac, worst)
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=DEV).tril(), float("-inf"))
    assert (lse - torch.logsumexp(scores, dim=-1)).abs().max().item() < 2e-2
    # the two kernels agree with each other as well
    out2, lse2 = flash_attention_forward(q, k, v, causal, scale, pingpong=False)
    frac, worst = _close(out, out2, rtol=2e-2, atol=0.02)
    assert frac == 0.0, ("vs two-pass", frac, worst)


def test_mlp_gelu_epilogue_backward():
    """gelu(x W1^T + b1) W2^T with the GELU derivative applied in the epilogue of the gradient GEMM (both the two-CTA and
    the one-CTA kernel, chosen by K) against fp32 autograd."""
    from oslo_b200.ops.gemm import mlp_gelu

    for rows, hid, ffn in ((4096, 1024, 4096), (512, 256, 512)):
        torch.manual_seed(81)
        x = (torch.randn(rows, hid, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
        w1 = (torch.randn(ffn, hid, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
        b1 = (torch.randn(ffn, device=DEV) * 0.1).to(torch.bfloat16).requires_grad_()
        w2 = (torch.randn(hid, ffn, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
        g = (torch.randn(rows, hid, device=DEV) * 0.5).to(torch.bfloat16)
        y = mlp_gelu(x, w1, b1, w2)
        y.backward(g)
        refs = [t.detach().float().requires_grad_() for t in (x, w1, b1, w2)]
        yr = torch.nn.functional.gelu(refs[0] @ refs[1].t() + refs[2], approximate="tanh") @ refs[3].t()
        yr.backward(g.float())
        frac, worst = _close(y, yr, rtol=2e-2, atol=0.02 * yr.abs().max().item())
        assert frac == 0.0, ("y", rows, frac, worst)
        for got, want, name in zip((x, w1, b1, w2), refs, ("dx", "dw1", "db1", "dw2")):
            frac, worst = _close(got.grad, want.grad, rtol=3e-2, atol=0.03 * want.grad.abs().max().item())
            assert frac < 1e-4, (name, rows, frac, worst)


def _close(a, b, rtol, atol):
    """Per-element check ``|a - b| <= atol + rtol * |b|`` (a single large element cannot hide errors elsewhere);
    returns the fraction of elements outside the bound and the worst excess, for the assertion message."""
    a, b = a.float(), b.float()
    excess = (a - b).abs() - (atol + rtol * b.abs())
    return (excess > 0).float().mean().item(), excess.max().item()


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True)])
def test_gemm_production_shape(a_t, b_t):
    """4096 x 3072 x 2048: 32 k-blocks (the 4-8 stage ring wraps and flips phase several times) and 384 / 768 tiles on
    148 persistent CTAs (each CTA runs 3-6 tiles, so both TMEM accumulator buffers and their phases are reused)."""
    from oslo_b200.ops.gemm import gemm

    torch.manual_seed(40)
    M, N, K = 4096, 3072, 2048
    a = (torch.randn((K, M) if a_t else (M, K), device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn((K, N) if b_t else (N, K), device=DEV) * 0.5).to(torch.bfloat16)
    A, B = (a.t() if a_t else a), (b.t() if b_t else b)
    ref = A.float() @ B.float().t()
    for bn in (0, 128):
        y = gemm(A, B, block_n=bn)
        # bf16 output rounding is 2^-9 relative; the fp32 accumulation error over K = 2048 is far below the atol
        frac, worst = _close(y, ref, rtol=1e-2, atol=0.05)
        assert frac == 0.0, (bn, frac, worst)


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_gemm_causal_modes_at_seq_2048(mode):
    """The three triangular work-skipping modes of the attention products at the sequence length the benchmark uses."""
    from oslo_b200.ops.gemm import gemm

    torch.manual_seed(41)
    s, hd = 2048, 128
    tril = torch.ones(s, s, device=DEV).tril()
    if mode == 1:  # scores = Q K^T, tiles above the diagonal skipped: compare the lower triangle only
        q = (torch.randn(2, s, hd, device=DEV) * 0.5).to(torch.bfloat16)
        k = (torch.randn(2, s, hd, device=DEV) * 0.5).to(torch.bfloat16)
        y = gemm(q, k, causal=1)
        ref = q.float() @ k.float().transpose(-1, -2)
        keep = tril.bool()  # skipped tiles are never written (they may hold anything, NaN included)
        frac, worst = _close(torch.where(keep, y.float(), torch.zeros_like(ref)), ref * tril, rtol=1e-2, atol=0.05)
    elif mode == 2:  # out = P V with lower-triangular P: reduce only over k <= row
        p = ((torch.rand(2, s, s, device=DEV) * tril) / 32).to(torch.bfloat16)
        v = (torch.randn(2, s, hd, device=DEV) * 0.5).to(torch.bfloat16)
        y = gemm(p, v.transpose(-1, -2), causal=2)
        ref = p.float() @ v.float()
        frac, worst = _close(y, ref, rtol=1e-2, atol=0.05)
    else:  # dV = P^T dO with P^T upper-triangular: reduce only over k >= row
        p = ((torch.rand(2, s, s, device=DEV) * tril) / 32).to(torch.bfloat16)
        do = (torch.randn(2, s, hd, device=DEV) * 0.5).to(torch.bfloat16)
        y = gemm(p.transpose(-1, -2), do.transpose(-1, -2), causal=3)
        ref = p.float().transpose(-1, -2) @ do.float()
        frac, worst = _close(y, ref, rtol=1e-2, atol=0.05)
    assert frac == 0.0, (mode, frac, worst)


def test_linear_gelu_fused_epilogue():
    from oslo_b200.ops.gemm import linear_gelu

    torch.manual_seed(42)
    x = (torch.randn(2, 512, 256, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(1024, 256, device=DEV) * 0.1).to(torch.bfloat16).requires_grad_()
    b = (torch.randn(1024, device=DEV) * 0.1).to(torch.bfloat16).requires_grad_()
    y = linear_gelu(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.gelu(F.linear(xr, wr, br), approximate="tanh")
    yr.backward(g.float())
    for got, want, name in ((y, yr, "y"), (x.grad, xr.grad, "dx"), (w.grad, wr.grad, "dw"), (b.grad, br.grad, "db")):
        frac, worst = _close(got, want, rtol=2e-2, atol=0.03 * want.abs().max().item())
        assert frac == 0.0, (name, frac, worst)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
def test_flash_attention_backward_two_groups(causal, hd):
    """The dK / dV kernel with two element-wise warp groups gives the gradients of the one-group kernel and of fp32."""
    from oslo_b200.ops import _lib
    from oslo_b200.ops.attention import attention, attention_reference, set_backward_groups

    torch.manual_seed(71)
    b, s, nh = 2, 768, 3  # 12 query tiles per key block: both groups and both buffer stages wrap several times
    qkv0 = (torch.randn(b, s, nh, 3, hd, device=DEV) * 0.7).to(torch.bfloat16)
    g = (torch.randn(b, s, nh * hd, device=DEV) * 0.5).to(torch.bfloat16)
    grads = {}
    try:
        for groups in (1, 2):
            set_backward_groups(groups, dq_groups=groups)
            qkv = qkv0.clone().requires_grad_()
            out = attention(qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :], causal=causal)
            out.backward(g)
            torch.cuda.synchronize()
            _lib.check_status()
            grads[groups] = qkv.grad.float()
    finally:
        set_backward_groups(2, dq_groups=1)  # the defaults
    ref_in = qkv0.float().requires_grad_()
    attention_reference(ref_in[..., 0, :], ref_in[..., 1, :], ref_in[..., 2, :], causal=causal).backward(g.float())
    tol = 0.03 * ref_in.grad.abs().max().item()
    for groups in (1, 2):
        frac, worst = _close(grads[groups], ref_in.grad, rtol=3e-2, atol=tol)
        assert frac < 1e-4, (groups, frac, worst)
    frac, worst = _close(grads[2], grads[1], rtol=1e-2, atol=0.01 * ref_in.grad.abs().max().item())
    assert frac < 1e-4, ("two groups vs one", frac, worst)


@pytest.mark.parametrize("causal", [True])
def test_flash_attention_seq_2048(causal):
    """Forward and backward at the benchmark's sequence length (16 key blocks per query block, causal skipping)."""
    from oslo_b200.ops.attention import attention, attention_reference

    torch.manual_seed(43)
    b, s, nh, hd = 1, 2048, 2, 128
    qkv = (torch.randn(b, s, nh, 3, hd, device=DEV) * 0.6).to(torch.bfloat16).requires_grad_()
    out = attention(qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :], causal=causal)
    g = torch.randn_like(out)
    out.backward(g)
    ref_in = qkv.detach().float().requires_grad_()
    ref = attention_reference(ref_in[..., 0, :], ref_in[..., 1, :], ref_in[..., 2, :], causal=causal)
    ref.backward(g.float())
    frac, worst = _close(out, ref, rtol=2e-2, atol=0.02)
    assert frac == 0.0, ("out", frac, worst)
    frac, worst = _close(qkv.grad, ref_in.grad, rtol=3e-2, atol=0.03 * ref_in.grad.abs().max().item())
    assert frac < 1e-4, ("dqkv", frac, worst)


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_two_cta(a_t, b_t):
    """The SM-pair kernel (tcgen05.mma.cta_group::2, 256 x 256 tiles) against fp32: all four operand layouts, a K that
    wraps the 6-stage ring several times, more tiles than SM pairs (both accumulator buffers reused), ragged M and N."""
    from oslo_b200.ops.gemm import gemm

    torch.manual_seed(44)
    M, N, K = 4096 + 128, 3072 + 64, 2048
    a = (torch.randn((K, M) if a_t else (M, K), device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn((K, N) if b_t else (N, K), device=DEV) * 0.5).to(torch.bfloat16)
    A, B = (a.t() if a_t else a), (b.t() if b_t else b)
    ref = A.float() @ B.float().t()
    y = gemm(A, B, two_cta=True)
    frac, worst = _close(y, ref, rtol=1e-2, atol=0.05)
    assert frac == 0.0, (frac, worst)


def test_gemm_two_cta_epilogues():
    from oslo_b200.ops.gemm import gemm

    torch.manual_seed(45)
    a = (torch.randn(1024, 512, device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn(768, 512, device=DEV) * 0.1).to(torch.bfloat16)
    bias = torch.randn(768, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float()
    frac, worst = _close(gemm(a, b, bias=bias, epilogue="bias", two_cta=True), ref, rtol=1e-2, atol=0.05)
    assert frac == 0.0, ("bias", frac, worst)
    aux = torch.empty(1024, 768, device=DEV, dtype=torch.bfloat16)
    y = gemm(a, b, bias=bias, epilogue="gelu", aux=aux, two_cta=True)
    frac, worst = _close(y, F.gelu(ref, approximate="tanh"), rtol=1e-2, atol=0.05)
    assert frac == 0.0, ("gelu", frac, worst)
    frac, worst = _close(aux, ref, rtol=1e-2, atol=0.05)
    assert frac == 0.0, ("aux", frac, worst)
    c = torch.randn(1024, 768, device=DEV, dtype=torch.bfloat16)
    c0 = c.float().clone()
    gemm(a, b, out=c, accumulate=True, two_cta=True)
    frac, worst = _close(c, c0 + a.float() @ b.float().t(), rtol=1e-2, atol=0.06)
    assert frac == 0.0, ("accumulate", frac, worst)
    a3 = (torch.randn(3, 512, 256, device=DEV) * 0.5).to(torch.float16)
    b3 = (torch.randn(3, 512, 256, device=DEV) * 0.5).to(torch.float16)
    frac, worst = _close(gemm(a3, b3, two_cta=True), a3.float() @ b3.float().transpose(-1, -2), rtol=1e-2, atol=0.05)
    assert frac == 0.0, ("batched fp16", frac, worst)


def test_lightseq_kernels_match_torch_paths():
    """Embedding (forward + backward, with and without dropout), int8 quantise / dequantise and the device-side top-k /
    top-p sampler against their plain-torch statements."""
    from oslo_b200.lightseq.kernels import filter_logits, ls_dequantize_int8, ls_embedding, ls_quantize_int8, sample_tokens

    torch.manual_seed(50)
    vocab, hid, seq = 500, 256, 48
    emb = (torch.randn(vocab, hid, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    pos = torch.randn(64, hid, device=DEV).to(torch.bfloat16)
    ids = torch.randint(1, vocab, (4, seq), device=DEV)
    ids[:, -5:] = 0  # padding
    out = ls_embedding(ids, emb, pos, step=3, padding_idx=0, scale=16.0, p=0.0)
    ref = torch.nn.functional.embedding(ids, emb.detach().float()) * 16.0 + pos[3 : 3 + seq].float()
    ref = ref.masked_fill((ids == 0).unsqueeze(-1), 0)
    assert _rel(out, ref) < 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    want = torch.zeros(vocab, hid, device=DEV)
    want.index_add_(0, ids.view(-1), (g.float() * 16.0).view(-1, hid) * (ids.view(-1, 1) != 0))
    assert _rel(emb.grad, want) < 2e-2
    # dropout: the kept pattern of the forward output is the mask that backward must recompute (zero positional table, so
    # that an output is zero only where it was dropped and never because a word and a position value cancel exactly)
    emb.grad = None
    out = ls_embedding(ids, emb, torch.zeros_like(pos), step=0, padding_idx=0, scale=1.0, p=0.3, training=True, seed=7)
    kept = out.detach() != 0
    frac = kept[ids != 0].float().mean().item()
    assert 0.6 < frac < 0.8, frac
    out.backward(torch.ones_like(out))
    want = torch.zeros(vocab, hid, device=DEV)
    want.index_add_(0, ids.view(-1), kept.view(-1, hid).float() / 0.7)
    assert _rel(emb.grad, want) < 2e-2
    # int8
    x = (torch.randn(4096, 129, device=DEV) * 2).to(torch.bfloat16)
    q, mask = ls_quantize_int8(x, 3.0, return_mask=True)
    qr = torch.round(x.float().clamp(-3, 3) * (127 / 3.0)).to(torch.int8)
    assert (q.int() - qr.int()).abs().max().item() <= 1 and torch.equal(mask, x.float().abs() > 3.0)
    assert _rel(ls_dequantize_int8(q, 3.0, torch.bfloat16), q.float() * (3.0 / 127)) < 1e-2
    # sampling: every draw lies in the filtered set, and the empirical distribution follows the renormalised probabilities
    logits = torch.randn(1, 2000, device=DEV) * 2
    for top_k, top_p in ((0, 1.0), (50, 1.0), (0, 0.8), (100, 0.5)):
        allowed = torch.isfinite(filter_logits(logits.float(), top_k, top_p))[0]
        draws = sample_tokens(logits.repeat(4096, 1), top_k, top_p).view(-1)
        assert bool(allowed[draws].all()), (top_k, top_p, int((~allowed[draws]).sum()))
        probs = filter_logits(logits.float(), top_k, top_p).softmax(-1)[0]
        top = probs.argmax()
        emp = (draws == top).float().mean().item()
        assert abs(emp - probs[top].item()) < 0.05, (top_k, top_p, emp, probs[top].item())
