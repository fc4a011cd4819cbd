"""Text generation for the in-tree causal language models: greedy, top-k / top-p sampling and beam search, with
n-gram blocking on the fused kernel and a key / value cache: the prompt is run once, after which every step feeds only
the newest token and attends over the cached keys and values (``oslo_b200.ops.attention.DecodeCache``).

A compact counterpart of LightSeq's inference engine entry points (oslo/lightseq2/inference/pywrapper/*, sampling and
beam-search kernels in inference/kernels/transformerKernels.cc.cu): the model forward runs on this repository's
training kernels; the decoding bookkeeping is vectorised torch code on the device (no host loop over hypotheses).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from oslo_b200.nn.ngram_repeat_block import NGramRepeatBlock
from oslo_b200.ops.attention import DecodeCache, decode_cache


def _logits(model, ids, cache: Optional[DecodeCache] = None):
    """Next-token logits.  With a cache only the tokens it has not seen yet are run through the model."""
    if cache is None:
        out = model(input_ids=ids)
    else:
        new = ids[:, cache.offset :]
        cache.begin_forward()
        with decode_cache(cache):
            out = model(input_ids=new)
        cache.advance(new.shape[1])
    logits = out.logits if hasattr(out, "logits") else out[0]
    return _whole_logits(model, logits[:, -1, :]).float()


def _whole_logits(model, last: torch.Tensor) -> torch.Tensor:
    """Tensor-parallel models whose head keeps the vocabulary sharded (for the vocab-parallel loss) return a slice of the
    logits; picking the next token needs all of them.  ``last``: ``[batch, vocab or a shard of it]``."""
    pc = getattr(model, "parallel_context", None)
    if pc is None or getattr(pc, "tensor_parallel_size", 1) == 1:
        return last
    base = getattr(model, "module", model)
    vocab = getattr(base, "orig_vocab_size", None) or base.config.vocab_size
    if last.shape[-1] >= vocab:
        return last[..., :vocab]
    from oslo_b200.distributed import ParallelMode, comm

    mode = pc.tensor_parallel_mode
    if mode == ParallelMode.TENSOR_1D:
        full = comm.all_gather(last.contiguous(), dim=-1, parallel_context=pc, parallel_mode=ParallelMode.TENSOR_1D)
    elif mode == ParallelMode.TENSOR_2D:
        from oslo_b200.parallel.tensor_parallel._ops_2d import gather_output_2d

        full = gather_output_2d(last.contiguous(), pc)
    elif mode == ParallelMode.TENSOR_2P5D:
        from oslo_b200.parallel.tensor_parallel._ops_2p5d import gather_output_2p5d

        full = gather_output_2p5d(last.contiguous(), pc)
    else:
        from oslo_b200.parallel.tensor_parallel._ops_3d import gather_output_3d

        full = gather_output_3d(last.contiguous(), pc)
    return full[..., :vocab]


def _filter(logits, top_k: int, top_p: float):
    if top_k and top_k > 0:
        kth = logits.topk(min(top_k, logits.shape[-1]), dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p and top_p < 1.0:
        sorted_logits, idx = logits.sort(dim=-1, descending=True)
        cum = sorted_logits.softmax(-1).cumsum(-1)
        drop = cum - sorted_logits.softmax(-1) > top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(1, idx, sorted_logits)
    return logits


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, max_new_tokens: int = 32, do_sample: bool = False, top_k: int = 0,
             top_p: float = 1.0, temperature: float = 1.0, num_beams: int = 1, no_repeat_ngram_size: int = 0,
             eos_token_id: Optional[int] = None, length_penalty: float = 1.0, pad_multiple: int = 1,
             use_cache: bool = True):
    """Returns ``[batch, prompt + new]`` token ids (best beam when ``num_beams > 1``).  ``use_cache=False`` re-runs the
    whole prefix every step (the reference behaviour for models whose attention does not go through ``oslo_b200.ops``)."""
    model.eval()
    pc = getattr(model, "parallel_context", None)
    if num_beams > 1 and use_cache and pc is not None and getattr(pc, "tensor_parallel_size", 1) > 1:
        from oslo_b200.distributed import ParallelMode as _PM

        if pc.tensor_parallel_mode != _PM.TENSOR_1D:
            # the N-D layouts split the batch over ranks, so a beam's parent may be cached on another rank: beams re-run
            # their prefix instead of reordering caches
            use_cache = False
    if num_beams > 1:
        return _beam_search(model, input_ids, max_new_tokens, num_beams, no_repeat_ngram_size, eos_token_id, length_penalty,
                            use_cache)
    ids = input_ids
    blocker = NGramRepeatBlock()
    done = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
    cache = DecodeCache() if use_cache else None
    for _ in range(max_new_tokens):
        logits = _logits(model, ids, cache) / max(temperature, 1e-6)
        if no_repeat_ngram_size > 0:
            logits = blocker(ids, logits.contiguous(), ids.shape[0], ids.shape[1] - 1, 1, no_repeat_ngram_size)
        if do_sample:
            from .kernels import sample_tokens

            nxt = sample_tokens(logits, top_k, top_p)  # the device kernel on CUDA (no vocabulary sort)
        else:
            nxt = logits.argmax(-1, keepdim=True)
        if eos_token_id is not None:
            nxt = torch.where(done.unsqueeze(1), torch.full_like(nxt, eos_token_id), nxt)
            done |= nxt.squeeze(1) == eos_token_id
        ids = torch.cat([ids, nxt], dim=1)
        if eos_token_id is not None and bool(done.all()):
            break
    return ids


def _beam_search(model, input_ids, max_new_tokens, beams, ngram, eos, length_penalty, use_cache=True):
    b, prompt = input_ids.shape
    dev = input_ids.device
    ids = input_ids.repeat_interleave(beams, dim=0)  # [b * beams, t]
    scores = torch.zeros(b, beams, device=dev)
    scores[:, 1:] = float("-inf")  # all beams start identical: keep one alive
    finished = torch.zeros(b * beams, dtype=torch.bool, device=dev)
    blocker = NGramRepeatBlock()
    cache = DecodeCache() if use_cache else None
    for _ in range(max_new_tokens):
        lp = F.log_softmax(_logits(model, ids, cache), dim=-1)
        if ngram > 0:
            lp = blocker(ids, lp.contiguous(), b, ids.shape[1] - 1, beams, ngram)
        vocab = lp.shape[-1]
        if eos is not None:
            # finished hypotheses may only extend with EOS at no cost
            frozen = torch.full_like(lp, float("-inf"))
            frozen[:, eos] = 0.0
            lp = torch.where(finished.unsqueeze(1), frozen, lp)
        cand = (scores.view(-1, 1) + lp).view(b, beams * vocab)
        top, idx = cand.topk(beams, dim=-1)
        src = idx // vocab + (torch.arange(b, device=dev) * beams).unsqueeze(1)
        tok = idx % vocab
        ids = torch.cat([ids[src.view(-1)], tok.view(-1, 1)], dim=1)
        if cache is not None:
            cache.reorder(src.view(-1))  # the surviving hypotheses keep the keys / values of the beams they extend
        scores = top
        if eos is not None:
            finished = finished[src.view(-1)] | (tok.view(-1) == eos)
            if bool(finished.all()):
                break
    new_len = ids.shape[1] - prompt
    final = scores / (max(new_len, 1) ** length_penalty)
    best = final.argmax(dim=-1) + torch.arange(b, device=dev) * beams
    return ids[best]
