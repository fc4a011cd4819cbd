"""LightSeq-interface models, CRF layer, weight export and the batching server (CPU)."""
import asyncio
import itertools
import os

import pytest
import torch


def test_transformer_trains_and_translates():
    from oslo_b200.lightseq import LSTransformer, get_config

    torch.manual_seed(0)
    cfg = get_config(model="transformer-base", vocab_size=40, padding_idx=0, max_seq_len=32, hidden_size=32,
                     intermediate_size=64, nhead=4, num_encoder_layer=2, num_decoder_layer=2, bos_id=1, eos_id=2)
    model = LSTransformer(cfg)
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    # copy task: the target is the source
    src = torch.randint(3, 40, (16, 6))
    trg_in = torch.cat([torch.full((16, 1), 1), src], dim=1)
    labels = torch.cat([src, torch.full((16, 1), 2)], dim=1)
    first = None
    for _ in range(150):
        loss, logits = model(src, trg_in, labels)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.3 * first, (first, loss.item())
    assert logits.shape == (16, 7, 40)
    model.eval()
    greedy = model.infer(src[:4], max_new_tokens=8)
    beam = model.infer(src[:4], max_new_tokens=8, beam_size=3)
    assert greedy.shape[0] == 4 and bool((greedy[:, 0] == 1).all())
    # a trained copy model reproduces most of the source with either search
    for out in (greedy, beam):
        n = min(out.shape[1] - 1, 6)
        assert (out[:, 1 : 1 + n] == src[:4, :n]).float().mean().item() > 0.7
    with pytest.raises(ValueError):
        get_config(model="transformer-huge")


def test_gpt_and_bert_models():
    from oslo_b200.lightseq import LSBert, LSGpt, get_config

    torch.manual_seed(1)
    cfg = get_config(vocab_size=50, padding_idx=0, max_seq_len=32, hidden_size=32, intermediate_size=64, nhead=4,
                     num_decoder_layer=2, num_encoder_layer=2, num_labels=3)
    gpt = LSGpt(cfg)
    ids = torch.randint(1, 50, (2, 10))
    out = gpt(ids, labels=ids)
    out.loss.backward()
    assert out.logits.shape == (2, 10, 50) and torch.isfinite(out.loss)
    gpt.eval()
    cached = gpt.infer(ids, max_new_tokens=4)
    full = gpt.infer(ids, max_new_tokens=4, use_cache=False)
    assert torch.equal(cached, full)  # the key / value cache (and the position offset of the embedding) change nothing
    bert = LSBert(cfg)
    loss, logits = bert(ids, labels=torch.tensor([0, 2]))
    loss.backward()
    assert logits.shape == (2, 3)


def _crf_brute_force(crf, e, mask):
    """All tag sequences of one example: log partition function and best path."""
    n = int(mask.sum())
    tags = crf.num_tags
    scores = {}
    for seq in itertools.product(range(tags), repeat=n):
        s = crf.start_transitions[seq[0]] + e[0, seq[0]]
        for t in range(1, n):
            s = s + crf.transitions[seq[t - 1], seq[t]] + e[t, seq[t]]
        scores[seq] = (s + crf.end_transitions[seq[-1]]).item()
    logz = torch.logsumexp(torch.tensor(list(scores.values())), 0).item()
    return scores, logz, max(scores, key=scores.get)


def test_crf_matches_brute_force():
    from oslo_b200.lightseq import LSCRFLayer

    torch.manual_seed(2)
    crf = LSCRFLayer(3)
    e = torch.randn(2, 5, 3)
    mask = torch.tensor([[1, 1, 1, 1, 1], [1, 1, 1, 0, 0]], dtype=torch.bool)
    tags = torch.tensor([[0, 1, 2, 1, 0], [2, 2, 1, 0, 0]])
    nll = crf(e, tags, mask, reduction="none")
    paths = crf.decode(e, mask)
    for i in range(2):
        scores, logz, best = _crf_brute_force(crf, e[i], mask[i])
        n = int(mask[i].sum())
        assert abs(nll[i].item() - (logz - scores[tuple(tags[i, :n].tolist())])) < 1e-4
        assert tuple(paths[i]) == best
    crf(e, tags, mask).backward()
    assert crf.transitions.grad is not None and torch.isfinite(crf.transitions.grad).all()


def test_export_roundtrip_plain_and_int8(tmp_path):
    from oslo_b200.lightseq import LSGpt, export_model, get_config, import_into, load_exported
    from oslo_b200.lightseq.export import read_header

    torch.manual_seed(3)
    cfg = get_config(vocab_size=64, padding_idx=0, max_seq_len=16, hidden_size=32, intermediate_size=64, nhead=4, num_decoder_layer=2)
    model = LSGpt(cfg).to(torch.bfloat16)
    path = os.path.join(tmp_path, "gpt.lsw")
    header = export_model(model, path, metadata={"note": "unit test"})
    assert header["config"]["hidden_size"] == 32 and read_header(path)[0]["metadata"]["note"] == "unit test"
    # the tied output projection is stored once
    assert "alias" in header["tensors"]["lm_head.weight"] or "alias" in header["tensors"]["embed_tokens.embeddings.weight"]
    state, _ = load_exported(path)
    for k, v in model.state_dict().items():
        assert torch.equal(state[k], v.cpu()), k
    fresh = LSGpt(cfg).to(torch.bfloat16)
    import_into(fresh, path)
    ids = torch.randint(1, 64, (2, 8))
    assert torch.equal(fresh(ids).logits, model(ids).logits)
    # int8: matrices within half a quantisation step, vectors exact, file a good deal smaller
    qpath = os.path.join(tmp_path, "gpt_int8.lsw")
    export_model(model.float(), qpath, quantize=True)
    qstate, qh = load_exported(qpath)
    assert qh["quantized"]
    for k, v in model.state_dict().items():
        e = qh["tensors"][k]
        if "alias" in e:
            continue
        if "clip" in e:
            assert (qstate[k] - v).abs().max().item() <= e["clip"] / 127 * 0.5 + 1e-6, k
        else:
            assert torch.equal(qstate[k], v), k
    raw, _ = load_exported(qpath, dequantize=False)
    assert raw["layers.0.attn.qkv.weight"].dtype == torch.int8
    export_model(model, os.path.join(tmp_path, "f32.lsw"))
    assert os.path.getsize(qpath) < 0.5 * os.path.getsize(os.path.join(tmp_path, "f32.lsw"))
    with open(os.path.join(tmp_path, "bad"), "wb") as f:
        f.write(b"not a weight file")
    with pytest.raises(ValueError):
        read_header(os.path.join(tmp_path, "bad"))


def test_dynamic_batcher_groups_requests():
    from oslo_b200.lightseq.serving import DynamicBatcher

    calls = []

    def fake_generate(ids, max_new_tokens=1):
        calls.append(tuple(ids.shape))
        return torch.cat([ids, ids[:, -1:].repeat(1, max_new_tokens) + 1], dim=1)

    async def main():
        b = DynamicBatcher(fake_generate, max_batch=4, max_wait_ms=50)
        res = await asyncio.gather(b.submit([1, 2, 3], max_new_tokens=2), b.submit([4, 5, 6], max_new_tokens=2),
                                   b.submit([7, 8], max_new_tokens=2), b.submit([9, 9, 9], max_new_tokens=1))
        await b.stop()
        return b, res

    b, res = asyncio.run(main())
    assert res[0][0] == [1, 2, 3, 4, 4] and res[1][0] == [4, 5, 6, 7, 7] and res[2][0] == [7, 8, 9, 9] and res[3][0] == [9, 9, 9, 10]
    assert res[0][1] == 2 and res[1][1] == 2  # the two same-length, same-settings prompts shared a batch
    assert sorted(calls) == [(1, 2), (1, 3), (2, 3)]
    assert b.requests == 4 and b.batches == 3


def test_http_server_generates():
    pytest.importorskip("fastapi")
    pytest.importorskip("httpx")
    from fastapi.testclient import TestClient

    from oslo_b200.lightseq import LSGpt, get_config
    from oslo_b200.lightseq.inference import generate
    from oslo_b200.lightseq.serving import create_app

    torch.manual_seed(4)
    cfg = get_config(vocab_size=50, padding_idx=0, max_seq_len=32, hidden_size=32, intermediate_size=64, nhead=4, num_decoder_layer=2)
    model = LSGpt(cfg).eval()
    with TestClient(create_app(model, max_batch=4, max_wait_ms=1)) as client:
        assert client.get("/health").json()["status"] == "ok"
        r = client.post("/generate", json={"input_ids": [[5, 6, 7], [8, 9, 10]], "max_new_tokens": 3})
        assert r.status_code == 200, r.text
        want = generate(model, torch.tensor([[5, 6, 7], [8, 9, 10]]), max_new_tokens=3).tolist()
        assert r.json()["output_ids"] == want
        assert client.post("/generate", json={"max_new_tokens": 3}).status_code == 422
        assert "oslo_requests_total 2" in client.get("/metrics").text
        # the inference protocol of Triton clients (KServe v2)
        assert client.get("/v2/health/ready").json() == {"ready": True} and client.get("/v2").json()["name"] == "oslo_b200"
        meta = client.get("/v2/models/oslo_b200").json()
        assert meta["inputs"][0] == {"name": "input_ids", "datatype": "INT64", "shape": [-1, -1]}
        assert client.get("/v2/models/other").status_code == 404
        body = {"id": "req-7", "inputs": [{"name": "input_ids", "datatype": "INT64", "shape": [2, 3], "data": [5, 6, 7, 8, 9, 10]}],
                "parameters": {"max_new_tokens": 3}}
        r = client.post("/v2/models/oslo_b200/infer", json=body)
        assert r.status_code == 200, r.text
        out = r.json()["outputs"][0]
        assert r.json()["id"] == "req-7" and out["shape"] == [2, 6] and out["data"] == [x for row in want for x in row]
        body["inputs"][0]["data"] = [[5, 6, 7], [8, 9, 10]]  # nested data is accepted too
        assert client.post("/v2/models/oslo_b200/versions/1/infer", json=body).json()["outputs"][0]["data"] == out["data"]
        assert client.post("/v2/models/oslo_b200/versions/2/infer", json=body).status_code == 404
        body["inputs"][0]["shape"] = [2, 4]
        assert client.post("/v2/models/oslo_b200/infer", json=body).status_code == 400
        assert client.post("/v2/models/oslo_b200/infer", json={"inputs": []}).status_code == 400


def test_cpu_gemms_match_torch():
    from oslo_b200.lightseq.cpu_gemm import gemm_u8s8s32, quantized_linear, sgemm

    torch.manual_seed(5)
    for ta, tb in itertools.product((False, True), repeat=2):
        a = torch.randn((37, 50) if ta else (50, 37))
        b = torch.randn((29, 37) if tb else (37, 29))
        want = (a.t() if ta else a) @ (b.t() if tb else b)
        got = sgemm(a, b, ta, tb)
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-4), (ta, tb, (got - want).abs().max())
        c0 = torch.randn(50, 29)
        got = sgemm(a, b, ta, tb, alpha=0.5, beta=2.0, out=c0.clone())
        assert torch.allclose(got, 0.5 * want + 2.0 * c0, rtol=1e-4, atol=1e-4)
        au = torch.randint(0, 256, (37, 50) if ta else (50, 37), dtype=torch.uint8)
        bs = torch.randint(-128, 128, (29, 37) if tb else (37, 29), dtype=torch.int8)
        comp = torch.randint(-1000, 1000, (29,), dtype=torch.int32)
        want_i = (au.t() if ta else au).to(torch.int64) @ (bs.t() if tb else bs).to(torch.int64) + comp
        got_i = gemm_u8s8s32(au, bs, ta, tb, compensation=comp)
        assert torch.equal(got_i.to(torch.int64), want_i), (ta, tb)
    # the quantised linear follows the fp32 one to quantisation accuracy
    x, w = torch.randn(64, 96), torch.randn(48, 96) * 0.2
    w_clip = float(w.abs().max())
    w_q = torch.round(w * (127.0 / w_clip)).to(torch.int8)
    y = quantized_linear(x, w_q, w_clip, x_clip=4.0, bias=torch.ones(48))
    ref = x.clamp(-4, 4) @ w.t() + 1.0
    assert (y - ref).abs().max().item() < 0.05 * ref.abs().max().item()


def test_layer_id_interface_with_flat_buffers():
    from oslo_b200.lightseq import registry as R
    from oslo_b200.lightseq.layers import LSLayerConfig, LSTransformerEncoderLayer

    torch.manual_seed(6)
    R.clear()
    assert R.create_transformer_encoder_layer(3, max_batch_tokens=64, max_seq_len=16, hidden_dim=32, num_heads=4,
                                              intermediate_size=64, is_pre_ln=True, activation_fn="gelu") == 0
    n = R.layer_param_numel("TransformerEncoderLayer", 3)
    flat_w, flat_g = torch.zeros(n), torch.zeros(n)
    before = [p.detach().clone() for p in R.get_layer("TransformerEncoderLayer", 3).parameters()]
    R.assign_layer_weight_grad(flat_w, flat_g, "TransformerEncoderLayer", 3)
    assert torch.equal(torch.cat([b.flatten() for b in before]), flat_w)  # the values moved into the flat buffer
    x = torch.randn(2, 5, 32)
    (y,) = R.transformer_encoder_layer_fw(3, x, torch.zeros(2, 5), True)
    (gx,) = R.transformer_encoder_layer_bw(3, torch.ones_like(y))
    # reference: the same module driven directly
    ref = LSTransformerEncoderLayer(LSLayerConfig(max_batch_tokens=64, max_seq_len=16, hidden_size=32, nhead=4, intermediate_size=64))
    ref.load_state_dict(R.get_layer("TransformerEncoderLayer", 3).state_dict())
    xr = x.clone().requires_grad_()
    yr = ref(xr)
    yr.backward(torch.ones_like(yr))
    assert torch.allclose(y, yr, atol=1e-6) and torch.allclose(gx, xr.grad, atol=1e-6)
    assert torch.allclose(flat_g, torch.cat([p.grad.flatten() for p in ref.parameters()]), atol=1e-6)
    # an update of the flat tensor is an update of the layer
    flat_w.sub_(0.1 * flat_g)
    (y2,) = R.transformer_encoder_layer_fw(3, x, None, False)
    assert not torch.allclose(y2, y)
    with pytest.raises(ValueError):
        R.assign_layer_weight_grad(torch.zeros(3), torch.zeros(3), "TransformerEncoderLayer", 3)
    R.clear()


def test_cli_train_validate_generate_export(tmp_path, capsys):
    from oslo_b200.lightseq import cli
    from oslo_b200.lightseq.export import read_header

    data = os.path.join(tmp_path, "pairs.tsv")
    g = torch.Generator().manual_seed(7)
    with open(data, "w") as f:
        for _ in range(48):
            s = torch.randint(3, 20, (5,), generator=g).tolist()
            f.write(" ".join(map(str, s)) + "\t" + " ".join(map(str, s)) + "\n")
    ckpt = os.path.join(tmp_path, "m.pt")
    assert cli.main(["train", "--data", data, "--save", ckpt, "--epochs", "30", "--batch-size", "16", "--lr", "0.003", "--hidden", "32",
                     "--heads", "4", "--layers", "1", "--max-len", "16", "--device", "cpu"]) == 0
    losses = [float(l.split("loss")[1]) for l in capsys.readouterr().out.splitlines() if l.startswith("epoch")]
    assert losses[-1] < 0.5 * losses[0]
    assert cli.main(["validate", "--load", ckpt, "--data", data, "--device", "cpu"]) == 0
    assert "perplexity" in capsys.readouterr().out
    src = os.path.join(tmp_path, "src.txt")
    with open(src, "w") as f:
        f.write("4 5 6 7 8\n9 10 11 12 13\n")
    assert cli.main(["generate", "--load", ckpt, "--input", src, "--beam", "2", "--max-new-tokens", "8", "--device", "cpu"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and all(l.replace(" ", "").isdigit() for l in lines if l)
    out = os.path.join(tmp_path, "m.lsw")
    assert cli.main(["export", "--load", ckpt, "--out", out, "--int8"]) == 0
    assert read_header(out)[0]["quantized"]


def test_lsflow_static_graph_matches_eager_and_reuses_memory():
    from oslo_b200.lightseq import lsflow
    from oslo_b200.lightseq.layers import LSLayerConfig, LSTransformerEncoderLayer

    torch.manual_seed(8)
    cfg = LSLayerConfig(max_batch_tokens=64, max_seq_len=16, hidden_size=32, intermediate_size=64, nhead=4, pre_layer_norm=True,
                        activation_fn="gelu")
    layers = [LSTransformerEncoderLayer(cfg).eval() for _ in range(3)]
    ctx = lsflow.Context()
    x = ctx.input("x", (64, 32))
    h = x
    for i, layer in enumerate(layers):
        h = lsflow.encoder_layer_graph(ctx, h, layer, f"layer{i}")
    ctx.build()
    # lifetimes let the planner fold 27 intermediates into far fewer bytes than their sum
    assert 0 < ctx.arena_bytes < 0.5 * ctx.naive_bytes, (ctx.arena_bytes, ctx.naive_bytes)
    for batch, seq in ((4, 16), (2, 8)):  # the second run is smaller than the declared maximum and reuses the arena
        inp = torch.randn(batch, seq, 32)
        want = inp
        with torch.no_grad():
            for layer in layers:
                want = layer(want)
        ptr = ctx.arena.data_ptr()
        (got,) = ctx.run({"x": inp.reshape(batch * seq, 32)}, [h], seq_len=seq)
        assert ctx.arena.data_ptr() == ptr
        assert torch.allclose(got.view(batch, seq, 32), want, atol=1e-5), (got.view(batch, seq, 32) - want).abs().max()
    with pytest.raises(ValueError):
        ctx.run({"x": torch.randn(65, 32)}, [h])
    with pytest.raises(RuntimeError):
        lsflow.AddOp(ctx, "late")(x, x)


def _ls_cfg(**kw):
    from oslo_b200.lightseq import get_config

    base = dict(vocab_size=97, hidden_size=32, intermediate_size=64, nhead=4, max_seq_len=48, padding_idx=0,
                num_encoder_layer=2, num_decoder_layer=2, num_labels=5)
    base.update(kw)
    return get_config(**base)


def test_lsflow_bert_and_bert_crf_match_the_eager_models_for_any_request_size():
    from oslo_b200.lightseq import LSBert, LSBertCrf, LSFlowBert, LSFlowBertCrf

    torch.manual_seed(0)
    for pre in (True, False):  # pre- and post-LayerNorm encoders
        model = LSBert(_ls_cfg(pre_layer_norm=pre, activation_fn="gelu")).eval()
        flow = LSFlowBert(model, max_batch=4, max_seq=16)
        mem = flow.memory(flow.ctx)
        assert mem["arena_bytes"] < mem["unplanned_bytes"] and mem["cache_bytes"] == 0
        arena = flow.ctx.arena.data_ptr()
        for b, s in ((4, 16), (1, 5), (3, 9)):
            ids = torch.randint(1, 97, (b, s))
            if b == 3:
                ids[0, 6:] = 0  # padded request
                ids[2, 4:] = 0
            with torch.no_grad():
                want = model(ids)
            got = flow.infer(ids)
            assert got.shape == want.shape and torch.allclose(got, want, atol=2e-5, rtol=1e-4), (pre, b, s)
        assert flow.ctx.arena.data_ptr() == arena  # no re-allocation between requests
        with pytest.raises(ValueError):
            flow.infer(torch.ones(5, 16, dtype=torch.long))
    tagger = LSBertCrf(_ls_cfg()).eval()
    # training direction: the CRF likelihood is differentiable through encoder and transitions
    ids = torch.randint(1, 97, (3, 10))
    ids[1, 7:] = 0
    tags = torch.randint(0, 5, (3, 10))
    loss, _ = tagger(ids, tags)
    loss.backward()
    assert tagger.crf.transitions.grad is not None and tagger.emission.weight.grad is not None
    flow = LSFlowBertCrf(tagger, max_batch=4, max_seq=12)
    paths = flow.infer(ids)
    assert paths == tagger.infer(ids) and [len(p) for p in paths] == [10, 7, 10]


def test_lsflow_gpt_decodes_incrementally_over_persistent_caches():
    from oslo_b200.lightseq import LSFlowGpt, LSGpt, generate

    torch.manual_seed(1)
    model = LSGpt(_ls_cfg(num_decoder_layer=3)).eval()
    flow = LSFlowGpt(model, max_batch=4, max_len=40)
    assert flow.memory(flow.ctx)["cache_bytes"] == 3 * 2 * 4 * 4 * 40 * 8 * 4  # layers x (k, v) x batch x heads x len x hd x fp32
    prompt = torch.randint(1, 97, (3, 7))
    out = flow.infer(prompt, max_new_tokens=12)
    want = generate(model, prompt, max_new_tokens=12, do_sample=False) if "do_sample" in generate.__code__.co_varnames else None
    if want is None:
        want = prompt
        with torch.no_grad():
            for _ in range(12):
                want = torch.cat([want, model(want).logits[:, -1].argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(out, want)
    assert flow.runs == 12  # one prompt run + eleven single-token runs
    # the logits of an incremental run equal those of a full-prefix forward
    flow.infer(prompt, max_new_tokens=1)
    nxt = model(prompt).logits[:, -1].argmax(-1, keepdim=True)
    inc = flow._step(nxt, 7)
    with torch.no_grad():
        full = model(torch.cat([prompt, nxt], dim=1)).logits[:, -1]
    assert torch.allclose(inc, full, atol=2e-5, rtol=1e-4)
    # sampling: reproducible under a seeded generator, stops at eos and pads after it
    g = torch.Generator().manual_seed(5)
    a = flow.infer(prompt, 10, top_k=8, top_p=0.9, temperature=0.8, generator=g)
    g = torch.Generator().manual_seed(5)
    b = flow.infer(prompt, 10, top_k=8, top_p=0.9, temperature=0.8, generator=g)
    assert torch.equal(a, b) and a.shape == (3, 17)
    eos = int(out[0, 9])
    stopped = flow.infer(prompt, 12, eos_token_id=eos)
    row = stopped[0, 7:].tolist()
    assert eos in row and all(t == 0 for t in row[row.index(eos) + 1:])
    with pytest.raises(ValueError):
        flow.infer(prompt, max_new_tokens=40)


def test_lsflow_transformer_translates_like_the_eager_model_greedy_and_beam():
    from oslo_b200.lightseq import LSFlowTransformer, LSTransformer

    torch.manual_seed(2)
    model = LSTransformer(_ls_cfg(activation_fn="relu")).eval()
    flow = LSFlowTransformer(model, max_batch=3, max_src=12, max_trg=16, max_beam=3)
    src = torch.randint(4, 97, (3, 9))
    src[1, 6:] = 0
    for beams in (1, 3):
        want = model.infer(src, max_new_tokens=10, beam_size=beams)
        got = flow.infer(src, max_new_tokens=10, beam_size=beams)
        assert torch.equal(got, want), beams
    mem = flow.memory()
    assert mem["cache_bytes"] > 0 and mem["arena_bytes"] < mem["unplanned_bytes"]
    with pytest.raises(ValueError):
        flow.infer(src, beam_size=4)


def test_vit_matches_a_conv_patch_embedding_and_its_graph():
    from oslo_b200.lightseq import LSFlowVit, LSVit

    torch.manual_seed(3)
    model = LSVit(_ls_cfg(num_labels=7, vocab_size=0), image_size=32, patch_size=8, channels=3).eval()
    x = torch.randn(3, 3, 32, 32)
    # the unfold + GEMM patch projection is a stride-8 convolution with the same weights
    conv = torch.nn.Conv2d(3, 32, 8, stride=8)
    with torch.no_grad():
        conv.weight.copy_(model.patch_proj.weight.view(32, 3, 8, 8))
        conv.bias.copy_(model.patch_proj.bias)
        want = conv(x).flatten(2).transpose(1, 2)
        got = model.patch_proj(model.patches(x))
    assert torch.allclose(got, want, atol=1e-5)
    with torch.no_grad():
        logits = model(x)
    assert logits.shape == (3, 7)
    loss, _ = model(x, torch.tensor([1, 2, 3]))
    loss.backward()
    assert model.pos_embed.grad is not None and model.cls_token.grad is not None
    flow = LSFlowVit(model, max_batch=4)
    assert torch.allclose(flow.infer(x), logits, atol=2e-5, rtol=1e-4)
    assert torch.allclose(flow.infer(x[:1]), logits[:1], atol=2e-5, rtol=1e-4)
    with pytest.raises(ValueError):
        model(torch.randn(1, 3, 16, 16))


def test_host_graph_executor_runs_the_same_graphs_in_one_native_call():
    """On the CPU the BERT / GPT / ViT graphs compile to a program for the C++ executor; results equal the node-by-node
    path and the eager models, including padding, incremental decoding and requests smaller than the plan."""
    from oslo_b200.lightseq import LSBert, LSFlowBert, LSFlowGpt, LSFlowVit, LSGpt, LSVit
    from oslo_b200.lightseq import lsflow as lf

    torch.manual_seed(4)
    bert = LSBert(_ls_cfg(pre_layer_norm=False)).eval()
    flow = LSFlowBert(bert, max_batch=4, max_seq=16)
    assert flow.native and flow.ctx._native is not None
    ids = torch.randint(1, 97, (3, 11))
    ids[1, 5:] = 0
    native = flow.infer(ids)
    flow.ctx._native = None  # node-by-node
    assert torch.allclose(native, flow.infer(ids), atol=1e-5)
    with torch.no_grad():
        assert torch.allclose(native, bert(ids), atol=2e-5, rtol=1e-4)

    gpt = LSGpt(_ls_cfg(num_decoder_layer=2)).eval()
    gflow = LSFlowGpt(gpt, max_batch=4, max_len=32)
    assert gflow.native
    prompt = torch.randint(1, 97, (2, 6))
    out = gflow.infer(prompt, max_new_tokens=9)
    want = prompt
    with torch.no_grad():
        for _ in range(9):
            want = torch.cat([want, gpt(want).logits[:, -1].argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(out, want)

    vit = LSVit(_ls_cfg(num_labels=3, vocab_size=0), image_size=16, patch_size=8).eval()
    vflow = LSFlowVit(vit, max_batch=2)
    x = torch.randn(2, 3, 16, 16)
    with torch.no_grad():
        assert vflow.native and torch.allclose(vflow.infer(x), vit(x), atol=2e-5, rtol=1e-4)

    # a graph with an operator the executor does not have keeps the node-by-node path
    from oslo_b200.lightseq import LSBertCrf, LSFlowBertCrf

    crf = LSFlowBertCrf(LSBertCrf(_ls_cfg()).eval(), max_batch=2, max_seq=8)
    assert crf.ctx.compile_native() is False and crf.infer(torch.randint(1, 97, (2, 8)))
    # errors come back as the failing node: a decoding step beyond the cache length
    with pytest.raises(RuntimeError, match="attn"):
        gflow.ctx.run({"ids": prompt.reshape(-1)}, [gflow.logits], seq_len=6, step=30)


def test_command_line_train_validate_generate_export(tmp_path, capsys):
    """The command-line workflow end to end on a toy reversal task: train, score, translate with beam search, export to
    int8 and read the export back."""
    import random

    from oslo_b200.lightseq import load_exported
    from oslo_b200.lightseq.cli import main

    rng = random.Random(0)
    data = tmp_path / "train.txt"
    with open(data, "w") as f:
        for _ in range(96):
            src = [rng.randint(4, 30) for _ in range(rng.randint(3, 6))]
            f.write(" ".join(map(str, src)) + "\t" + " ".join(map(str, reversed(src))) + "\n")
    model = str(tmp_path / "m.pt")
    common = ["--device", "cpu"]
    assert main(["train", "--data", str(data), "--save", model, "--epochs", "3", "--batch-size", "16", "--lr", "3e-3", "--vocab-size", "32",
                 "--hidden", "32", "--heads", "4", "--layers", "1", "--max-len", "12", *common]) == 0
    losses = [float(line.split()[-1]) for line in capsys.readouterr().out.splitlines() if line.startswith("epoch")]
    assert len(losses) == 3 and losses[-1] < losses[0]
    assert main(["validate", "--load", model, "--data", str(data), *common]) == 0
    assert "perplexity" in capsys.readouterr().out
    src = tmp_path / "in.txt"
    src.write_text("5 6 7\n8 9 10 11\n")
    assert main(["generate", "--load", model, "--input", str(src), "--beam", "2", "--max-new-tokens", "6", *common]) == 0
    lines = capsys.readouterr().out.splitlines()  # one line per source sentence (empty when the model stops at once)
    assert len(lines) == 2 and all(tok.isdigit() for line in lines for tok in line.split())
    out = str(tmp_path / "m.osl")
    assert main(["export", "--load", model, "--out", out, "--int8", *common]) == 0
    state, header = load_exported(out)
    assert header["quantized"] and len(state) == len(header["tensors"]) > 5
