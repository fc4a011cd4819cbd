"""Python entry points of the LightSeq-specific kernels (``csrc/lightseq_sm100a.cu``), each with a plain-torch path that is
used on CPU and serves as the numerics reference in the tests.

* ``ls_embedding``       token lookup x scale + positional row + dropout with padding rows zeroed, forward and backward
                         (LightSeq ``transformer_embedding_layer_fw/bw``, oslo/lightseq2/csrc/kernels/cuda/embedding_kernels.cu)
* ``ls_quantize_int8`` / ``ls_dequantize_int8``   symmetric int8 with a clip maximum and the clipped-element mask
                         (oslo/lightseq2/csrc/kernels/cuda/quantize_kernels.cu)
* ``sample_tokens``      top-k / top-p sampling of the next token on the device, no vocabulary sort
                         (oslo/lightseq2/inference/kernels/transformerKernels.cc.cu)
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from oslo_b200.ops import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and _lib.has_cuda_kernels() and t.dtype in _DT


class _LSEmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, emb, pos, step, pad, scale, p, seed, offset):
        b, s = ids.shape
        h = emb.shape[1]
        ids_c = ids.contiguous().view(-1)
        out = torch.empty(b * s, h, dtype=emb.dtype, device=emb.device)
        rc = _lib.cuda_lib().oslo_ls_embedding_forward(
            _lib.ptr(ids_c), _lib.ptr(emb), _lib.ptr(pos), _lib.ptr(out), ctypes.c_longlong(b * s), ctypes.c_int(s), ctypes.c_int(h),
            ctypes.c_int(step), ctypes.c_int(pad), ctypes.c_float(scale), ctypes.c_float(p), ctypes.c_ulonglong(seed),
            ctypes.c_ulonglong(offset), ctypes.c_int(_DT[emb.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ls_embedding_forward failed ({rc})")
        ctx.save_for_backward(ids_c)
        ctx.meta = (emb.shape, emb.dtype, pad, scale, p, seed, offset)
        return out.view(b, s, h)

    @staticmethod
    def backward(ctx, g):
        (ids_c,) = ctx.saved_tensors
        shape, dtype, pad, scale, p, seed, offset = ctx.meta
        g2 = g.contiguous().view(-1, shape[1])
        acc = torch.zeros(shape, dtype=torch.float32, device=g.device)
        rc = _lib.cuda_lib().oslo_ls_embedding_backward(
            _lib.ptr(ids_c), _lib.ptr(g2), _lib.ptr(acc), ctypes.c_longlong(ids_c.numel()), ctypes.c_int(shape[1]), ctypes.c_int(pad),
            ctypes.c_float(scale), ctypes.c_float(p), ctypes.c_ulonglong(seed), ctypes.c_ulonglong(offset), ctypes.c_int(_DT[dtype]),
            ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ls_embedding_backward failed ({rc})")
        return None, acc.to(dtype), None, None, None, None, None, None, None


_offset = 0


def ls_embedding(ids: torch.Tensor, emb: torch.Tensor, pos: torch.Tensor, step: int = 0, padding_idx: int = 0,
                 scale: float = 1.0, p: float = 0.0, training: bool = True, seed: Optional[int] = None) -> torch.Tensor:
    """``dropout(emb[ids] * scale + pos[step : step + seq])`` with the rows of padding tokens zeroed; ``ids``: ``[batch, seq]``,
    ``pos``: ``[max_positions, hidden]`` in the dtype of ``emb``."""
    global _offset
    p = float(p) if training else 0.0
    if _cuda(emb) and emb.shape[1] % 8 == 0 and pos.dtype == emb.dtype and pos.is_contiguous() and emb.is_contiguous():
        _offset += 1
        sd = int(torch.initial_seed() if seed is None else seed) & ((1 << 63) - 1)
        return _LSEmbeddingFn.apply(ids, emb, pos, int(step), int(padding_idx), float(scale), p, sd, _offset)
    s = ids.shape[1]
    x = torch.nn.functional.embedding(ids, emb) * scale + pos[step : step + s].to(emb.dtype)
    x = x.masked_fill((ids == padding_idx).unsqueeze(-1), 0)
    return torch.nn.functional.dropout(x, p, training) if p > 0 else x


def ls_quantize_int8(x: torch.Tensor, clip_max: float, return_mask: bool = False):
    """``round(clamp(x, -clip_max, clip_max) * 127 / clip_max)`` as int8 (and the ``|x| > clip_max`` mask)."""
    if _cuda(x):
        xc = x.contiguous()
        q = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
        mask = torch.empty(xc.shape, dtype=torch.uint8, device=x.device) if return_mask else None
        rc = _lib.cuda_lib().oslo_ls_quantize(_lib.ptr(xc), _lib.ptr(q), _lib.ptr(mask), ctypes.c_longlong(xc.numel()),
                                              ctypes.c_float(clip_max), ctypes.c_int(_DT[x.dtype]), ctypes.c_int(_lib.num_sms()),
                                              _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ls_quantize failed ({rc})")
        return (q, mask.bool()) if return_mask else q
    xf = x.float()
    q = torch.round(xf.clamp(-clip_max, clip_max) * (127.0 / clip_max)).to(torch.int8)
    return (q, xf.abs() > clip_max) if return_mask else q


def ls_dequantize_int8(q: torch.Tensor, clip_max: float, dtype=torch.float32) -> torch.Tensor:
    if q.is_cuda and _lib.has_cuda_kernels() and dtype in _DT:
        qc = q.contiguous()
        x = torch.empty(qc.shape, dtype=dtype, device=q.device)
        rc = _lib.cuda_lib().oslo_ls_dequantize(_lib.ptr(qc), _lib.ptr(x), ctypes.c_longlong(qc.numel()), ctypes.c_float(clip_max),
                                                ctypes.c_int(_DT[dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ls_dequantize failed ({rc})")
        return x
    return (q.float() * (clip_max / 127.0)).to(dtype)


def sample_tokens(logits: torch.Tensor, top_k: int = 0, top_p: float = 1.0, temperature: float = 1.0,
                  generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """One token id per row of ``logits [rows, vocab]`` drawn from the temperature-scaled distribution restricted to the
    ``top_k`` largest logits and then to the nucleus of mass ``top_p`` inside them.  Returns ``[rows, 1]`` int64."""
    rows, v = logits.shape
    if _cuda(logits):
        lc = logits.contiguous()
        u = torch.rand(rows, device=logits.device, generator=generator, dtype=torch.float32)
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
        rc = _lib.cuda_lib().oslo_ls_sample(_lib.ptr(lc), _lib.ptr(u), _lib.ptr(out), ctypes.c_int(rows), ctypes.c_int(v),
                                            ctypes.c_int(int(top_k)), ctypes.c_float(float(top_p)), ctypes.c_float(float(temperature)),
                                            ctypes.c_int(_DT[logits.dtype]), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ls_sample failed ({rc})")
        return out.view(rows, 1)
    return torch.multinomial(filter_logits(logits.float() / temperature, top_k, top_p).softmax(-1), 1, generator=generator)


def filter_logits(logits: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """The torch statement of the sampling filter: top-k first, then the nucleus inside what is left."""
    if top_k and 0 < top_k < logits.shape[-1]:
        kth = logits.topk(top_k, dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p and top_p < 1.0:
        sorted_logits, idx = logits.sort(dim=-1, descending=True)
        probs = sorted_logits.softmax(-1)
        cum = probs.cumsum(-1)
        drop = cum - probs >= top_p  # keep the smallest prefix whose mass reaches top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(1, idx, sorted_logits)
    return logits
