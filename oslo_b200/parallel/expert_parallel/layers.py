"""Router, experts and the front / behind blocks of an expert-parallel mixture-of-experts feed-forward layer.

Data path of one MoE layer over an expert group of ``ep`` ranks with ``E`` experts (``E/ep`` local), ``S`` local tokens:

    logits  = x Wg (fp32)                              [S, E]
    routing = top-1 / top-2 choice, capacity C, slot = expert * C + position (or dropped)
    buf     = dispatch(x, slot)                        [E, C, h]         (row gather by index)
    buf     = all_to_all(buf)                          [E/ep, ep * C, h]
    h1      = buf W1_e^T + b1_e   (batched tcgen05 GEMM over local experts)      <- front block returns this
    (the model applies its activation)
    h2      = h1 W2_e^T + b2_e
    out     = combine(all_to_all^-1(h2), gate weights, slot)                    <- behind block returns this

The load-balancing loss of every layer is kept in ``link.l_aux`` and added to the model loss by the wrapper
(the reference computes it and drops it: oslo/torch/nn/parallel/expert_parallel/layers.py:499-501).
Parity: layers.py:121-632 and experts.py:5-43 of the reference.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from oslo_b200.distributed import ParallelMode, comm
from oslo_b200.ops import moe as moe_ops
from oslo_b200.ops.gemm import gemm, supported


def _gumbel(shape, device):
    u = torch.rand(shape, device=device).clamp_(1e-9, 1 - 1e-9)
    return -torch.log(-torch.log(u))


def _capacity(num_tokens: int, num_experts: int, factor: float, min_capacity: int) -> int:
    return max(int(math.ceil(num_tokens / num_experts * factor)), int(min_capacity))


class TopKGate(nn.Module):
    """fp32 router.  Returns ``(l_aux, slot [S, k] int32, weight [S, k], capacity)``."""

    def __init__(self, model_dim, num_experts, k=1, capacity_factor=1.0, eval_capacity_factor=1.0, min_capacity=4,
                 noisy_gate_policy: Optional[str] = None, drop_tokens=True, use_rts=True):
        super().__init__()
        if k not in (1, 2):
            raise ValueError("only top-1 and top-2 gating are supported")
        if noisy_gate_policy not in (None, "Jitter", "RSample"):
            raise ValueError(f"unknown noisy_gate_policy {noisy_gate_policy}")
        self.wg = nn.Linear(model_dim, num_experts, bias=False).float()
        self.num_experts, self.k = num_experts, k
        self.capacity_factor, self.eval_capacity_factor = capacity_factor, eval_capacity_factor
        self.min_capacity = min_capacity
        self.noisy_gate_policy, self.drop_tokens, self.use_rts = noisy_gate_policy, drop_tokens, use_rts

    def forward(self, x):
        E = self.num_experts
        xf = x.float()
        if self.noisy_gate_policy == "Jitter" and self.training:
            xf = xf * torch.empty_like(xf).uniform_(1 - 1e-2, 1 + 1e-2)
        logits = F.linear(xf, self.wg.weight.float())
        S = logits.shape[0]
        gates = F.softmax(logits, dim=1)
        factor = self.capacity_factor if self.training else self.eval_capacity_factor
        if self.k == 1:
            pick = logits + _gumbel(logits.shape, logits.device) if (self.noisy_gate_policy == "RSample" and self.training) else gates
            idx1 = pick.argmax(dim=1)
            C = _capacity(S, E, factor, self.min_capacity)
            mask1 = F.one_hot(idx1, E).to(gates.dtype)
            l_aux = torch.sum(gates.mean(0) * mask1.mean(0)) * E
            choice = idx1.unsqueeze(1)
            if self.use_rts and self.drop_tokens and self.training:
                # random token selection: when an expert overflows, keep a random subset instead of the first C
                prio = torch.rand(S, device=logits.device)
                key = idx1.double() + (1.0 - prio.double()) * 0.5
                order = torch.argsort(key)
                ranks = torch.empty_like(order)
                counts = torch.bincount(idx1, minlength=E)
                starts = torch.cumsum(counts, 0) - counts
                ranks[order] = torch.arange(S, device=logits.device) - starts[idx1[order]]
                choice = torch.where((ranks < C).unsqueeze(1), choice, torch.full_like(choice, -1))
            weights = gates.gather(1, idx1.unsqueeze(1))
        else:
            idx1 = gates.argmax(dim=1)
            noise = _gumbel(logits.shape, logits.device) if self.training else 0.0
            idx2 = (logits + noise).masked_fill(F.one_hot(idx1, E).bool(), float("-inf")).argmax(dim=1)
            C = _capacity(S, E, factor * 2, self.min_capacity)
            mask1 = F.one_hot(idx1, E).to(gates.dtype)
            l_aux = torch.mean(gates.mean(0) * mask1.mean(0)) * E * E
            choice = torch.stack([idx1, idx2], dim=1)
            weights = gates.gather(1, choice)
        if not self.drop_tokens:
            pc = getattr(self, "parallel_context", None)
            cnt = torch.bincount(choice[choice >= 0].reshape(-1), minlength=E).max()
            if pc is not None:
                cnt = comm.all_reduce(cnt.clone(), op=torch.distributed.ReduceOp.MAX, parallel_context=pc,
                                      parallel_mode=ParallelMode.GLOBAL)
            C = max(C, int(cnt.item()))
        pos, _ = moe_ops.positions(choice.to(torch.int32), E)
        kept = (choice >= 0) & (pos < C)
        slot = torch.where(kept, choice.to(torch.int32) * C + pos, torch.full_like(pos, -1))
        weights = weights * kept
        if self.k == 2:
            weights = weights / weights.sum(1, keepdim=True).clamp(min=torch.finfo(weights.dtype).eps)
        return l_aux, slot, weights, C


class Experts(nn.Module):
    """``E_local`` independent linears stored stacked: weight ``[E_local, out, in]`` (or ``[E_local, in, out]`` when
    ``reversed``), bias ``[E_local, out]``; applied as one batched tcgen05 GEMM."""

    def __init__(self, num_local_experts, in_features, out_features, bias=True, reversed=False, dtype=None, device=None):
        super().__init__()
        self.num_local_experts, self.reversed = num_local_experts, reversed
        shape = (num_local_experts, in_features, out_features) if reversed else (num_local_experts, out_features, in_features)
        self.weight = nn.Parameter(torch.empty(shape, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(num_local_experts, out_features, dtype=dtype, device=device)) if bias else None
        for p in self.parameters():
            p.oslo_expert_param = True

    def forward(self, x):  # x: [E_local, T, in]
        w = self.weight.transpose(1, 2) if self.reversed else self.weight  # [E_local, out, in]
        y = _BatchedLinear.apply(x, w)
        if self.bias is not None:
            y = y + self.bias.unsqueeze(1)
        return y


class _BatchedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        if supported(x, w) and x.shape[-1] % 8 == 0 and w.shape[1] % 8 == 0:
            return gemm(x, w)
        return torch.matmul(x, w.transpose(1, 2))

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gy = gy.contiguous()
        if supported(gy, w) and x.shape[-1] % 8 == 0 and w.shape[1] % 8 == 0 and x.shape[1] % 8 == 0:
            gx = gemm(gy, w.transpose(1, 2))
            gw = gemm(gy.transpose(1, 2), x.transpose(1, 2))
        else:
            gx = torch.matmul(gy, w)
            gw = torch.matmul(gy.transpose(1, 2), x)
        return gx, gw


class MoELink:
    """State shared by the front and behind block of one MoE layer during a forward pass."""

    def __init__(self):
        self.slot = self.weight = None
        self.capacity = 0
        self.l_aux = None
        self.in_shape = None


def _all_to_all_experts(buf, ep, e_local, C, pc, inverse=False):
    """[E, C, h] <-> [E_local, ep * C, h] over the expert group."""
    h = buf.shape[-1]
    if ep == 1:
        return buf.view(e_local, C, h)
    if not inverse:
        out = _AllToAll.apply(buf.view(ep * e_local * C, h), pc)  # chunks by destination rank -> by source rank
        return out.view(ep, e_local, C, h).transpose(0, 1).reshape(e_local, ep * C, h)
    src = buf.view(e_local, ep, C, h).transpose(0, 1).reshape(ep * e_local * C, h)
    return _AllToAll.apply(src, pc).view(ep * e_local, C, h)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pc):
        ctx.pc = pc
        return comm.all_to_all(x.contiguous(), parallel_context=pc, parallel_mode=ParallelMode.EXPERT)

    @staticmethod
    def backward(ctx, g):
        return comm.all_to_all(g.contiguous(), parallel_context=ctx.pc, parallel_mode=ParallelMode.EXPERT), None


class ExpertParallelFrontBlock(nn.Module):
    def __init__(self, gate: TopKGate, experts: Experts, link: MoELink, parallel_context, ep_size, num_local_experts,
                 skip_bias_add=False, residual: Optional[nn.Module] = None):
        super().__init__()
        self.gate, self.experts = gate, experts
        self.link, self.parallel_context = link, parallel_context
        self.ep_size, self.num_local_experts = ep_size, num_local_experts
        self.skip_bias_add = skip_bias_add
        # Residual-MoE (reference layers.py:402-461): a dense copy of the replaced linear runs beside the experts and a
        # learned 2-way softmax mixes the two results per token
        self.residual = residual
        self.residual_mix = None
        if residual is not None:
            w = next(residual.parameters())
            self.residual_mix = nn.Linear(gate.wg.weight.shape[1], 2, dtype=w.dtype, device=w.device)

    # Libraries peek at ``module.weight`` / ``module.bias`` of the linear this block replaced (dtype checks before a cast):
    # answer with the experts' tensors.
    @property
    def weight(self):
        return self.experts.weight

    @property
    def bias(self):
        return self.experts.bias

    def forward(self, x):
        link = self.link
        link.in_shape = x.shape
        tokens = x.reshape(-1, x.shape[-1])
        l_aux, slot, weight, C = self.gate(tokens)
        link.l_aux, link.slot, link.weight, link.capacity = l_aux, slot, weight, C
        E = self.ep_size * self.num_local_experts
        from . import fused

        link.fused = fused.available(tokens, self.ep_size)
        if link.fused:
            # the dispatch kernel stores every token row straight into its expert's buffer on the owning GPU
            buf = fused.PeerDispatch.apply(tokens, slot, self.parallel_context, self.ep_size, self.num_local_experts, C)
        else:
            buf = moe_ops.dispatch(tokens, slot, E * C)
            buf = _all_to_all_experts(buf, self.ep_size, self.num_local_experts, C, self.parallel_context)
        out = self.experts(buf)
        link.residual_rows = 0
        if self.residual is not None:
            # the dense intermediate rides behind the expert rows, so whatever the model applies between the two
            # linears of its MLP (activation, dropout) covers both; the behind block splits them again
            inter = self.residual(tokens)
            if isinstance(inter, tuple):  # a skip_bias_add linear hands its bias back: the experts have none to add it to
                inter = inter[0] if inter[1] is None else inter[0] + inter[1]
            link.residual_weight = torch.softmax(self.residual_mix(tokens).float(), dim=-1)
            link.expert_shape = out.shape
            link.residual_rows = inter.shape[0]
            out = torch.cat([out.reshape(-1, out.shape[-1]), inter.to(out.dtype)], dim=0)
        return (out, None) if self.skip_bias_add else out


class ExpertParallelBehindBlock(nn.Module):
    def __init__(self, experts: Experts, link: MoELink, parallel_context, ep_size, num_local_experts, skip_bias_add=False,
                 residual: Optional[nn.Module] = None):
        super().__init__()
        self.experts = experts
        self.link, self.parallel_context = link, parallel_context
        self.ep_size, self.num_local_experts = ep_size, num_local_experts
        self.skip_bias_add = skip_bias_add
        self.residual = residual  # dense copy of the replaced linear (Residual-MoE)

    # Libraries peek at ``module.weight`` / ``module.bias`` of the linear this block replaced (dtype checks before a cast):
    # answer with the experts' tensors.
    @property
    def weight(self):
        return self.experts.weight

    @property
    def bias(self):
        return self.experts.bias

    def forward(self, x):  # x: [E_local, ep * C, ffn]  (+ the dense rows behind it under Residual-MoE)
        link = self.link
        dense = None
        rows = getattr(link, "residual_rows", 0)
        if rows:
            dense = x[x.shape[0] - rows :]
            x = x[: x.shape[0] - rows].view(link.expert_shape)
        out = self.experts(x)
        if getattr(link, "fused", False):
            from . import fused

            y = fused.PeerCombine.apply(out, link.weight, link.slot, self.parallel_context, self.ep_size, self.num_local_experts,
                                        link.capacity)
        else:
            out = _all_to_all_experts(out, self.ep_size, self.num_local_experts, link.capacity, self.parallel_context, inverse=True)
            y = moe_ops.combine(out.reshape(-1, out.shape[-1]), link.weight.to(out.dtype), link.slot)
        if dense is not None:
            if self.residual is None:
                raise RuntimeError("the front block produced a dense residual but this block has no residual module")
            r = self.residual(dense)
            r = r[0] + r[1] if isinstance(r, tuple) and r[1] is not None else (r[0] if isinstance(r, tuple) else r)
            w = link.residual_weight
            y = (y.float() * w[:, 0:1] + r.float() * w[:, 1:2]).to(y.dtype)
        y = y.view(*link.in_shape[:-1], y.shape[-1])
        return (y, None) if self.skip_bias_add else y
