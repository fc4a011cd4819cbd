"""``ExpertParallel(module, parallel_context, num_dec_experts=..., top_k=2, ...)``: turns chosen FFN layers into
mixtures of experts sharded over the EXPERT group.

The mapped first / second FFN linears of every selected layer are replaced by an ``ExpertParallelFrontBlock`` /
``ExpertParallelBehindBlock`` pair (see ``layers.py``).  Expert ``e`` (global id) lives on expert-rank
``e // (E / ep)``; its weights are drawn from a generator seeded by ``(seed, layer, e)`` so the same experts arise for
any ``ep``.  The load-balancing loss of all MoE layers is added to ``output.loss`` with ``aux_loss_coef``.

Gradient handling: dense (non-expert) parameters are replicated over the expert group, so their gradients are
averaged over it at the end of backward — unless a data-parallel wrapper / ZeRO over an overlaying DATA group does
that already (``sync_dense_grads=False``).  Expert gradients are divided by ``ep`` because every rank's loss is a
mean over its own tokens only.

``deparallelize()`` gathers all experts to every rank; ``save_extra_states`` writes them to ``ep_extra_states.bin``.
Parity: oslo/torch/nn/parallel/expert_parallel/expert_parallel.py:30-598.
"""
from __future__ import annotations

import copy
import os
from typing import Dict, Optional, Union

import torch
import torch.nn as nn

from oslo_b200.distributed import ParallelMode, comm
from oslo_b200.parallel.utils import ParallelWrapper, add_wrapper, get_parallel_context

from .layers import ExpertParallelBehindBlock, ExpertParallelFrontBlock, Experts, MoELink, TopKGate
from .mapping import Behind, ExpertParallelMapping, Front


def _is_conv1d(m):
    return m.__class__.__name__ == "Conv1D"


class ExpertParallel(ParallelWrapper):
    #: before the tensor-parallel wrapper (priority 0): experts are built from the whole feed-forward linears, and the
    #: tensor-parallel wrapper then leaves everything inside an expert block alone
    parallelism_priority = -1

    def __init__(self, module: nn.Module, parallel_context=None, num_enc_experts: Union[int, dict, None] = None,
                 num_dec_experts: Union[int, dict, None] = None, top_k: int = 2, capacity_factor_train: float = 1.0,
                 capacity_factor_eval: float = 1.0, min_capacity: int = 4, noisy_policy: Optional[str] = None,
                 use_rts: bool = True, drop_tokens: bool = True, use_residual: bool = False,
                 extra_states_path: Optional[str] = None, mapping: Optional[dict] = None, aux_loss_coef: float = 0.01,
                 sync_dense_grads: Optional[bool] = None, seed: int = 1234):
        super().__init__()
        self.module = module
        self.parallel_context = pc = get_parallel_context(module, parallel_context)
        self.num_experts = {"enc": num_enc_experts, "dec": num_dec_experts}
        self.top_k, self.min_capacity = top_k, min_capacity
        self.capacity_factor_train, self.capacity_factor_eval = capacity_factor_train, capacity_factor_eval
        self.noisy_policy, self.use_rts, self.drop_tokens = noisy_policy, use_rts, drop_tokens
        self.use_residual = use_residual
        self.extra_states_path = extra_states_path
        self.aux_loss_coef = aux_loss_coef
        self.seed = seed
        self.mapping = ExpertParallelMapping(mapping)
        self.ep_size = pc.get_world_size(ParallelMode.EXPERT) if pc.is_initialized(ParallelMode.EXPERT) else 1
        self.ep_rank = pc.get_local_rank(ParallelMode.EXPERT) if pc.is_initialized(ParallelMode.EXPERT) else 0
        if self.ep_size > 1 and pc.pipeline_parallel_size > 1:
            # Two pipeline stages x two expert ranks (four gloo ranks) did not finish a step: the experts' exchange and the
            # pipeline's point-to-point schedule wait on each other.  Refused up front rather than left to hang.
            raise NotImplementedError("expert parallelism (size > 1) cannot be combined with pipeline parallelism; "
                                      "use tensor and / or data parallelism around the experts")
        if sync_dense_grads is None:
            sync_dense_grads = not pc.topology.expert_overlay
        self.sync_dense_grads = sync_dense_grads and self.ep_size > 1
        self.links: Dict[str, MoELink] = {}
        self._dense_params, self._callback_queued = [], False
        add_wrapper(module, ParallelMode.EXPERT, self)

    # ------------------------------------------------------------------ forward
    def forward(self, *args, **kwargs):
        out = self.module(*args, **kwargs)
        loss = getattr(out, "loss", None)
        if loss is not None and self.links and self.aux_loss_coef:
            aux = sum(l.l_aux for l in self.links.values() if l.l_aux is not None)
            out.aux_loss = aux
            out.loss = loss + self.aux_loss_coef * aux.to(loss.dtype)
        return out

    def _experts_for(self, stack: str, layer_idx: int) -> int:
        spec = self.num_experts[stack]
        if spec is None:
            return 0
        if isinstance(spec, int):
            return spec
        if isinstance(spec, dict):
            return int(spec.get(layer_idx, spec.get(str(layer_idx), 0)))
        if isinstance(spec, (list, tuple)):
            return int(spec[layer_idx]) if layer_idx < len(spec) else 0
        raise TypeError("num_*_experts must be an int, a dict {layer: n} or a list")

    # -------------------------------------------------------------- parallelize
    @torch.no_grad()
    def parallelize(self):
        module, pc = self.module, self.parallel_context
        module.parallel_context = pc
        replaced = {}
        for name, child in list(module.named_modules()):
            hit = self.mapping.match(module, name)
            if hit is None or not (isinstance(child, nn.Linear) or _is_conv1d(child)):
                continue
            info, layer_idx, stack = hit
            E = self._experts_for(stack, layer_idx)
            if E == 0:
                continue
            if E % self.ep_size:
                raise ValueError(f"{E} experts cannot be split over an expert group of {self.ep_size}")
            e_local = E // self.ep_size
            key = f"{stack}.{layer_idx}"
            link = self.links.setdefault(key, MoELink())
            conv = _is_conv1d(child)
            w = child.weight
            in_f, out_f = (w.shape[0], w.shape[1]) if conv else (w.shape[1], w.shape[0])
            experts = Experts(e_local, in_f, out_f, bias=getattr(child, "bias", None) is not None, reversed=conv,
                              dtype=w.dtype, device=w.device)
            std = getattr(getattr(module, "config", None), "initializer_range", 0.02)
            role = 0 if isinstance(info, Front) else 1
            for le in range(e_local):
                ge = self.ep_rank * e_local + le
                gen = torch.Generator().manual_seed(self.seed + 1000003 * layer_idx + 7919 * ge + role)
                experts.weight.data[le].copy_(torch.randn(experts.weight.shape[1:], generator=gen).mul_(std).to(w.dtype))
            skip = getattr(child, "skip_bias_add", False)
            if isinstance(info, Front):
                gate = TopKGate(in_f, E, self.top_k, self.capacity_factor_train, self.capacity_factor_eval,
                                self.min_capacity, self.noisy_policy, self.drop_tokens, self.use_rts)
                ggen = torch.Generator().manual_seed(self.seed + 31 * layer_idx + 17)
                gate.wg.weight.data.copy_(torch.randn(gate.wg.weight.shape, generator=ggen).mul_(std))
                gate.wg.to(w.device)
                gate.parallel_context = pc
                new = ExpertParallelFrontBlock(gate, experts, link, pc, self.ep_size, e_local, skip_bias_add=skip,
                                               residual=copy.deepcopy(child) if self.use_residual else None)
            else:
                new = ExpertParallelBehindBlock(experts, link, pc, self.ep_size, e_local, skip_bias_add=skip,
                                                residual=copy.deepcopy(child) if self.use_residual else None)
            parent = module
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], new)
            replaced[name] = new
        ep = self.ep_size
        for p in module.parameters():
            if getattr(p, "oslo_expert_param", False):
                if ep > 1:
                    p.register_post_accumulate_grad_hook(self._scale_expert_grad)
            elif self.sync_dense_grads and p.requires_grad:
                self._dense_params.append(p)
                p.register_post_accumulate_grad_hook(self._dense_hook)
        if self.sync_dense_grads:
            src = pc.get_ranks_in_group(ParallelMode.EXPERT)[0]
            for p in self._dense_params:
                comm.broadcast(p.data, src=src, parallel_context=pc, parallel_mode=ParallelMode.EXPERT)

    def _scale_expert_grad(self, p):
        p.grad.div_(self.ep_size)

    def _dense_hook(self, p):
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._reduce_dense_grads)

    def _reduce_dense_grads(self):
        self._callback_queued = False
        pc = self.parallel_context
        by_dtype = {}
        for p in self._dense_params:
            if p.grad is not None:
                by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
        for gs in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in gs])
            comm.all_reduce(flat, parallel_context=pc, parallel_mode=ParallelMode.EXPERT)
            flat.div_(self.ep_size)
            off = 0
            for g in gs:
                g.copy_(flat[off : off + g.numel()].view_as(g))
                off += g.numel()

    # ------------------------------------------------------------ checkpoints
    def _gather_experts(self, t: torch.Tensor) -> torch.Tensor:
        if self.ep_size == 1:
            return t
        return comm.all_gather(t.contiguous(), dim=0, parallel_context=self.parallel_context, parallel_mode=ParallelMode.EXPERT)

    def merge_state_dict_hook(self, state: dict) -> dict:
        """Merged checkpoints hold ALL experts of every MoE layer (collective over the expert group)."""
        out = dict(state)
        for key, p in self.module.state_dict(keep_vars=True).items():
            if getattr(p, "oslo_expert_param", False):
                out[key] = self._gather_experts(p.data).cpu()
        return out

    def save_extra_states(self, save_directory: str):
        """``ep_extra_states.bin``: every expert and router tensor, keys prefixed ``module.`` (as the reference)."""
        state = {}
        for key, p in self.module.state_dict(keep_vars=True).items():
            if getattr(p, "oslo_expert_param", False):
                state["module." + key] = self._gather_experts(p.data).cpu()
            elif ".gate." in key:
                state["module." + key] = p.detach().cpu()
        if self.parallel_context.get_global_rank() == 0:
            os.makedirs(save_directory, exist_ok=True)
            torch.save(state, os.path.join(save_directory, "ep_extra_states.bin"))
        return state

    @torch.no_grad()
    def deparallelize(self):
        """Give every rank all experts (``ep`` becomes 1 for this wrapper's layers)."""
        if self.ep_size == 1:
            return
        for m in self.module.modules():
            if isinstance(m, Experts):
                w = self._gather_experts(m.weight.data)
                m.weight = nn.Parameter(w)
                m.weight.oslo_expert_param = True
                if m.bias is not None:
                    m.bias = nn.Parameter(self._gather_experts(m.bias.data))
                    m.bias.oslo_expert_param = True
                m.num_local_experts = w.shape[0]
            if isinstance(m, (ExpertParallelFrontBlock, ExpertParallelBehindBlock)):
                m.num_local_experts *= m.ep_size
                m.ep_size = 1
        self.ep_size = 1
