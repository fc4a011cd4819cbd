"""Inference models on the static-graph runtime: BERT classifier, BERT + CRF tagger, GPT generator, translation
Transformer.

Counterpart of the reference's lsflow models (oslo/lightseq2/csrc/models/{bert,bert_crf,gpt,transformer}.cc with
``model_base.h``: each builds its layer graph once against maximum shapes, then ``Infer()`` feeds token ids and reads the
output buffers).  A model here wraps the trained ``nn.Module`` (parameters are bound, not copied), declares its graph in
:class:`oslo_b200.lightseq.lsflow.Context`, and after ``build()`` every request of any batch size / length up to the
maxima runs through the same planned arena; generators keep their key / value caches in persistent buffers and run one
token per step after the prompt.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from . import lsflow as lf


def _embed(ctx: lf.Context, ids: lf.Variable, emb, name: str) -> lf.Variable:
    cfg = emb.config
    return lf.EmbeddingOp(ctx, name, emb.embeddings.weight, emb.pos_embeddings, cfg.padding_idx, math.sqrt(cfg.hidden_size))(ids)


def _mask_of(ids: torch.Tensor, padding_idx: int) -> Optional[torch.Tensor]:
    pad = ids == padding_idx
    return pad if bool(pad.any()) else None


class _FlowModel:
    """Shared plumbing: device / dtype of the wrapped module, memory figures of the plan."""

    def __init__(self, module: torch.nn.Module, max_batch: int, max_seq: int):
        p = next(module.parameters())
        self.module, self.device, self.dtype = module.eval(), p.device, p.dtype
        self.max_batch, self.max_seq = max_batch, max_seq

    def memory(self, *contexts: lf.Context) -> dict:
        return {"arena_bytes": sum(c.arena_bytes for c in contexts), "unplanned_bytes": sum(c.naive_bytes for c in contexts),
                "cache_bytes": sum(c.persistent_bytes for c in contexts)}

    def _check(self, ids: torch.Tensor):
        if ids.dim() != 2:
            raise ValueError("token ids are [batch, seq]")
        if ids.shape[0] > self.max_batch or ids.shape[1] > self.max_seq:
            raise ValueError(f"request {tuple(ids.shape)} exceeds the planned maximum ({self.max_batch}, {self.max_seq})")


def _encoder_graph(ctx: lf.Context, encoder, max_tokens: int):
    ids = ctx.input("ids", (max_tokens,), torch.int64)
    x = _embed(ctx, ids, encoder.embed_tokens, "embed")
    for i, layer in enumerate(encoder.layers):
        x = lf.encoder_layer_graph(ctx, x, layer, f"enc{i}")
    if encoder.layer_norm is not None:
        n = encoder.layer_norm
        x = lf.LayerNormOp(ctx, "enc.ln", n.weight, n.bias, n.eps)(x)
    return ids, x


class LSFlowBert(_FlowModel):
    """:class:`oslo_b200.lightseq.models.LSBert` as a planned graph: ``infer(input_ids) -> logits [batch, labels]``."""

    def __init__(self, model, max_batch: int = 8, max_seq: int = 128):
        super().__init__(model, max_batch, max_seq)
        ctx = self.ctx = lf.Context(self.device)
        _, x = _encoder_graph(ctx, model.encoder, max_batch * max_seq)
        pooled = lf.ActivationOp(ctx, "pool.tanh", "tanh")(lf.SelectTokenOp(ctx, "pool", 0)(x))
        self.logits = lf.LinearOp(ctx, "classifier", model.classifier.weight, model.classifier.bias)(pooled)
        ctx.build()
        self.native = ctx.compile_native()  # host fp32 graphs run as one call into the C++ executor

    @torch.no_grad()
    def infer(self, input_ids: torch.Tensor) -> torch.Tensor:
        self._check(input_ids)
        b, s = input_ids.shape
        mask = _mask_of(input_ids, self.module.config.padding_idx)
        (out,) = self.ctx.run({"ids": input_ids.reshape(-1)}, [self.logits], seq_len=s, padding_mask=mask)
        return out.clone()


class LSFlowBertCrf(_FlowModel):
    """:class:`oslo_b200.lightseq.models.LSBertCrf` as a planned graph: ``infer(input_ids) -> list of tag paths``."""

    def __init__(self, model, max_batch: int = 8, max_seq: int = 128):
        super().__init__(model, max_batch, max_seq)
        ctx = self.ctx = lf.Context(self.device)
        _, x = _encoder_graph(ctx, model.encoder, max_batch * max_seq)
        self.emissions = lf.LinearOp(ctx, "emission", model.emission.weight, model.emission.bias)(x)
        self.tags = lf.CRFDecodeOp(ctx, "crf", model.crf)(self.emissions)
        ctx.build()

    @torch.no_grad()
    def infer(self, input_ids: torch.Tensor) -> List[List[int]]:
        self._check(input_ids)
        b, s = input_ids.shape
        mask = _mask_of(input_ids, self.module.config.padding_idx)
        (tags,) = self.ctx.run({"ids": input_ids.reshape(-1)}, [self.tags], seq_len=s, padding_mask=mask)
        tags = tags.view(b, s).tolist()
        return [[t for t in row if t >= 0] for row in tags]


class LSFlowVit(_FlowModel):
    """:class:`oslo_b200.lightseq.models.LSVit` as a planned graph: ``infer(pixels) -> logits [batch, labels]``.  The
    patch extraction and the class-token / position add run before the graph (they are one reshape and one add); the
    patch projection, the encoder and the head are graph nodes."""

    def __init__(self, model, max_batch: int = 8):
        super().__init__(model, max_batch, model.num_patches + 1)
        ctx = self.ctx = lf.Context(self.device)
        seq = model.num_patches + 1
        x = ctx.input("tokens", (max_batch * seq, model.config.hidden_size), self.dtype)
        for i, layer in enumerate(model.layers):
            x = lf.encoder_layer_graph(ctx, x, layer, f"enc{i}")
        n = model.layer_norm
        x = lf.LayerNormOp(ctx, "ln", n.weight, n.bias, n.eps)(x)
        cls = lf.SelectTokenOp(ctx, "cls", 0)(x)
        self.logits = lf.LinearOp(ctx, "head", model.classifier.weight, model.classifier.bias)(cls)
        ctx.build()
        self.native = ctx.compile_native()

    @torch.no_grad()
    def infer(self, pixels: torch.Tensor) -> torch.Tensor:
        if pixels.shape[0] > self.max_batch:
            raise ValueError(f"batch {pixels.shape[0]} exceeds the planned maximum {self.max_batch}")
        tokens = self.module.embed(pixels)
        b, s, h = tokens.shape
        (out,) = self.ctx.run({"tokens": tokens.reshape(b * s, h).contiguous()}, [self.logits], seq_len=s)
        return out.clone()


def _pick(logits: torch.Tensor, top_k: int, top_p: float, temperature: float, generator) -> torch.Tensor:
    if top_k == 1 or (top_k == 0 and top_p >= 1.0 and temperature == 0.0):
        return logits.argmax(-1, keepdim=True)
    from .kernels import sample_tokens

    return sample_tokens(logits.float(), top_k, top_p, max(temperature, 1e-6), generator)


class LSFlowGpt(_FlowModel):
    """:class:`oslo_b200.lightseq.models.LSGpt` as a planned graph with persistent key / value caches.

    ``infer(input_ids, max_new_tokens, top_k=1, ...)``: the prompt runs once (``seq = prompt length``, ``step = 0``); every
    later run feeds the newest token only (``seq = 1``, ``step = tokens so far``).  ``top_k = 1`` is greedy."""

    def __init__(self, model, max_batch: int = 8, max_len: int = 256):
        super().__init__(model, max_batch, max_len)
        ctx = self.ctx = lf.Context(self.device)
        ids = ctx.input("ids", (max_batch * max_len,), torch.int64)
        x = _embed(ctx, ids, model.embed_tokens, "embed")
        for i, layer in enumerate(model.layers):
            x = lf.encoder_layer_graph(ctx, x, layer, f"dec{i}", cache=(max_batch, max_len))
        n = model.layer_norm
        x = lf.LayerNormOp(ctx, "ln_f", n.weight, n.bias, n.eps)(x)
        last = lf.SelectTokenOp(ctx, "last", -1)(x)
        self.logits = lf.LinearOp(ctx, "lm_head", model.lm_head.weight, None)(last)
        ctx.build()
        self.native = ctx.compile_native()  # host fp32 graphs run as one call into the C++ executor
        self.runs = 0

    def _step(self, ids: torch.Tensor, step: int) -> torch.Tensor:
        self.runs += 1
        (out,) = self.ctx.run({"ids": ids.reshape(-1)}, [self.logits], seq_len=ids.shape[1], step=step)
        return out

    @torch.no_grad()
    def infer(self, input_ids: torch.Tensor, max_new_tokens: int = 32, top_k: int = 1, top_p: float = 1.0, temperature: float = 1.0,
              eos_token_id: Optional[int] = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        self._check(input_ids)
        b, s = input_ids.shape
        if s + max_new_tokens > self.max_seq:
            raise ValueError(f"{s} prompt + {max_new_tokens} new tokens exceed the cache length {self.max_seq}")
        out = input_ids
        done = torch.zeros(b, dtype=torch.bool, device=input_ids.device)
        logits = self._step(input_ids, 0)
        pad = self.module.config.padding_idx
        for t in range(max_new_tokens):
            nxt = _pick(logits, top_k, top_p, temperature, generator).view(b, 1)
            if eos_token_id is not None:
                nxt = torch.where(done[:, None], torch.full_like(nxt, pad), nxt)
                done = done | (nxt.view(-1) == eos_token_id)
            out = torch.cat([out, nxt], dim=1)
            if t == max_new_tokens - 1 or (eos_token_id is not None and bool(done.all())):
                break
            logits = self._step(nxt, s + t)
        return out


class LSFlowTransformer(_FlowModel):
    """:class:`oslo_b200.lightseq.models.LSTransformer` as two planned graphs: the encoder runs once per source batch,
    its output is projected into every decoder layer's memory keys / values, and the decoder then runs one target token
    per step over its self-attention caches.  Greedy or beam search (caches reordered to follow the surviving beams)."""

    def __init__(self, model, max_batch: int = 8, max_src: int = 128, max_trg: int = 128, max_beam: int = 4):
        super().__init__(model, max_batch, max_src)
        self.max_trg, self.max_beam = max_trg, max_beam
        enc = self.enc_ctx = lf.Context(self.device)
        _, self.enc_out = _encoder_graph(enc, model.encoder, max_batch * max_src)
        enc.build()
        self.native = enc.compile_native()  # the encoder; the decoder's memory attention stays node by node
        rows = max_batch * max_beam
        dec = self.dec_ctx = lf.Context(self.device)
        ids = dec.input("ids", (rows * max_trg,), torch.int64)
        x = _embed(dec, ids, model.decoder.embed_tokens, "embed")
        self.cross: List[lf.CrossAttentionOp] = []
        self.cached: List[lf.CachedAttentionOp] = []
        for i, layer in enumerate(model.decoder.layers):
            x, cross = lf.decoder_layer_graph(dec, x, layer, f"dec{i}", rows, max_trg, max_src)
            self.cross.append(cross)
        self.cached = [n for n in dec._nodes if isinstance(n, lf.CachedAttentionOp)]
        if model.decoder.layer_norm is not None:
            n = model.decoder.layer_norm
            x = lf.LayerNormOp(dec, "dec.ln", n.weight, n.bias, n.eps)(x)
        last = lf.SelectTokenOp(dec, "last", -1)(x)
        self.logits = lf.LinearOp(dec, "proj", model.decoder.output_projection.weight, None)(last)
        dec.build()

    def memory(self):
        return super().memory(self.enc_ctx, self.dec_ctx)

    @torch.no_grad()
    def infer(self, src_tokens: torch.Tensor, max_new_tokens: int = 64, beam_size: int = 1, length_penalty: float = 0.6) -> torch.Tensor:
        self._check(src_tokens)
        if beam_size > self.max_beam or max_new_tokens + 1 > self.max_trg:
            raise ValueError("beam size or target length exceeds the planned maximum")
        cfg = self.module.config
        b, s = src_tokens.shape
        mask = _mask_of(src_tokens, cfg.padding_idx)
        (enc,) = self.enc_ctx.run({"ids": src_tokens.reshape(-1)}, [self.enc_out], seq_len=s, padding_mask=mask)
        enc = enc.view(b, s, -1)
        if beam_size > 1:
            enc = enc.repeat_interleave(beam_size, dim=0)
            mask = mask.repeat_interleave(beam_size, dim=0) if mask is not None else None
        for op in self.cross:
            op.encode_memory(enc, mask)
        n = b * beam_size
        dev = src_tokens.device
        out = torch.full((n, 1), cfg.bos_id, dtype=torch.long, device=dev)
        scores = torch.zeros(b, beam_size, device=dev)
        if beam_size > 1:
            scores[:, 1:] = -1e9
        done = torch.zeros(n, dtype=torch.bool, device=dev)
        for t in range(max_new_tokens):
            (logits,) = self.dec_ctx.run({"ids": out[:, -1].contiguous()}, [self.logits], seq_len=1, step=t)
            logp = torch.log_softmax(logits.float(), dim=-1)
            logp[done] = -1e9
            logp[done, cfg.padding_idx] = 0.0
            if beam_size == 1:
                nxt = logp.argmax(-1)
            else:
                v = logp.shape[-1]
                cand = (scores.view(-1, 1) + logp).view(b, beam_size * v)
                scores, idx = cand.topk(beam_size, dim=-1)
                parent = (idx // v + torch.arange(b, device=dev).unsqueeze(1) * beam_size).view(-1)
                nxt = (idx % v).view(-1)
                out, done = out[parent], done[parent]
                for op in self.cached:
                    op.reorder(parent)
            out = torch.cat([out, nxt[:, None]], dim=1)
            done = done | (nxt == cfg.eos_id)
            if bool(done.all()):
                break
        if beam_size > 1:
            lengths = (out != cfg.padding_idx).sum(-1).view(b, beam_size).float()
            best = (scores / lengths.pow(length_penalty)).argmax(-1)
            out = out.view(b, beam_size, -1)[torch.arange(b, device=dev), best]
        return out


__all__ = ["LSFlowBert", "LSFlowBertCrf", "LSFlowGpt", "LSFlowTransformer", "LSFlowVit"]
