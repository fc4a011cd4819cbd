"""LM head + cross-entropy without materialising the full logits.

``linear_cross_entropy(hidden [T, H], weight [V, H], targets [T])`` walks the tokens in chunks: each chunk's logits
(``chunk x V``) are produced by the GEMM, reduced to the loss by the cross-entropy kernel, turned into ``dlogits`` in place
and immediately consumed by the two gradient GEMMs (``d hidden`` for the chunk, ``d weight`` accumulated in fp32 or in the
weight's dtype through the GEMM's accumulate epilogue).  Peak memory for the head drops from ``T x V`` logits (+ their
gradient) to ``chunk x V``: 1.6 GB + 1.6 GB at 16384 x 50304 bf16 become 2 x 0.4 GB at the default chunk of 4096.
The gradients are computed during the forward pass (the loss is a mean over tokens, so each chunk's contribution is
known up to the scalar ``grad_output`` that the backward multiplies in), which is what makes the logits disposable.

Counterpart of the "optionally fused with the LM-head GEMM" form of the vocab-parallel cross-entropy of the reference's
loss functions (oslo/torch/nn/modules/functional/loss.py); with a tensor-parallel vocabulary each chunk goes through
:func:`oslo_b200.ops.loss.vocab_parallel_cross_entropy`, so the statistics are exchanged per chunk.
"""
from __future__ import annotations

from typing import Optional

import torch

from oslo_b200.distributed import ParallelMode


def _chunk_loss_and_grad(logits, targets, pc, mode, ignore_index, orig_vocab):
    """Sum of the token losses of one chunk and d(sum)/d(logits), through the vocab-parallel kernel path."""
    from .loss import vocab_parallel_cross_entropy

    leaf = logits.detach().requires_grad_(True)
    with torch.enable_grad():
        # a view of the leaf: the CUDA kernel overwrites its input with the gradient, which it refuses to do to a leaf
        per_token = vocab_parallel_cross_entropy(leaf.view_as(leaf), targets, pc, mode, ignore_index, orig_vocab)
        total = per_token.float().sum()
    (g,) = torch.autograd.grad(total, leaf)
    return total.detach(), g


class _LinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, chunk, ignore_index, pc, mode, orig_vocab):
        from .gemm import gemm, supported

        T, H = hidden.shape
        n_valid = (targets != ignore_index).sum().clamp(min=1)
        d_hidden = torch.empty_like(hidden)
        d_weight = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        total = torch.zeros((), dtype=torch.float32, device=hidden.device)
        use_kernel = supported(hidden, weight) and H % 8 == 0 and weight.shape[0] % 8 == 0
        for s in range(0, T, chunk):
            h = hidden[s : s + chunk]
            t = targets[s : s + chunk]
            logits = gemm(h, weight) if use_kernel else h @ weight.t()
            loss_sum, g = _chunk_loss_and_grad(logits, t, pc, mode, ignore_index, orig_vocab)
            del logits
            total += loss_sum
            g = g.to(hidden.dtype)
            if use_kernel:
                gemm(g, weight.t(), out=d_hidden[s : s + chunk])       # [c, V] x [V, H]
                d_weight += gemm(g.t(), h.t()).float()                  # [V, c] x [c, H]
            else:
                d_hidden[s : s + chunk] = g @ weight
                d_weight += (g.t() @ h).float()
            del g
        if pc is not None and pc.get_world_size(mode) > 1:
            # every rank holds the contribution of its vocabulary shard to d hidden: sum them (what the backward of a
            # column-parallel head does)
            import torch.distributed as dist

            dist.all_reduce(d_hidden, group=pc.get_group(mode))
        inv = 1.0 / n_valid.float()
        ctx.save_for_backward(d_hidden, d_weight, inv)
        ctx.mark_non_differentiable(targets)
        return total * inv

    @staticmethod
    def backward(ctx, grad_out):
        d_hidden, d_weight, inv = ctx.saved_tensors
        scale = (grad_out.float() * inv)
        gh = (d_hidden.float() * scale).to(d_hidden.dtype) if ctx.needs_input_grad[0] else None
        gw = (d_weight * scale).to(d_hidden.dtype) if ctx.needs_input_grad[1] else None
        return gh, gw, None, None, None, None, None, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, chunk_size: int = 4096,
                         ignore_index: int = -100, parallel_context=None, parallel_mode=ParallelMode.TENSOR_1D,
                         orig_vocab_size: Optional[int] = None) -> torch.Tensor:
    """Mean over the non-ignored tokens of ``cross_entropy(hidden @ weight^T, targets)``; ``hidden`` may have leading batch
    dimensions.  ``weight`` may be this rank's vocabulary shard (pass the parallel context); ``orig_vocab_size`` masks the
    padded tail of a padded vocabulary."""
    h2 = hidden.reshape(-1, hidden.shape[-1])
    return _LinearCEFn.apply(h2, weight, targets.reshape(-1), int(chunk_size), ignore_index, parallel_context, parallel_mode,
                             orig_vocab_size)


__all__ = ["linear_cross_entropy"]
