"""``PipelineParallel(module, parallel_context, memory_computation_balance=1.0, num_micro_batches=1)``:
pipeline parallelism with a 1F1B schedule over point-to-point sends (NCCL on GPUs, gloo on CPU).

The reference offloads every sub-module call to its owner through RPC round trips
(oslo/torch/nn/parallel/pipeline_parallel/pipeline_parallel.py:161-474); here the model is cut into contiguous
stages and only stage boundaries communicate.  The public contract is kept:

    for ind, out in wrapped(**batch):       # one iteration per micro-batch
        out.loss.backward()

On the last stage ``out.loss`` is the micro-batch loss (already divided by the number of micro-batches); on other
stages it is a placeholder whose ``backward()`` does nothing — those stages run their backward passes inside the
generator when the gradients arrive, following 1F1B: stage ``s`` of ``P`` does ``min(P-1-s, M)`` warm-up forwards, then
alternates one forward and one backward, then drains.

Overlap: the receive of micro-batch ``i + 1``'s activation is posted (``irecv``) as soon as micro-batch ``i``'s has
arrived, i.e. before the stage computes ``i``, so the transfer runs under the compute.  Gradients travel on a second
communicator over the same ranks: point-to-point operations between one pair of ranks execute in issue order on one
stream, and an early-posted activation receive must never sit in front of a gradient send to the same neighbour.

A model provides its decomposition through ``pipeline_units()`` (a list of :class:`PipeUnit`); ``nn.Sequential`` works
out of the box.  Parameters used by units on several stages (tied embeddings) are kept on each of them and their
gradients are summed at the end of the batch.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from oslo_b200.distributed import ParallelMode
from oslo_b200.distributed.p2p import P2P
from oslo_b200.parallel.utils import ParallelWrapper, add_wrapper, get_parallel_context
from oslo_b200.transformers.constants import BATCH_DIMENSIONS_PP

from .partitioner import ModelPartitioner, PipeUnit, sequential_units


class _RemoteLoss:
    """Stands in for the loss on stages that do not compute it."""

    def backward(self, *a, **k):
        return None

    def item(self):
        return float("nan")

    def detach(self):
        return self


class PipelineOutput:
    def __init__(self, loss=None, logits=None):
        self.loss, self.logits = loss, logits


class PipelineParallel(ParallelWrapper):
    parallelism_priority = 99

    def __init__(self, module: nn.Module, parallel_context=None, memory_computation_balance: float = 1.0,
                 num_micro_batches: int = 1):
        super().__init__()
        self.module = module
        self.parallel_context = pc = get_parallel_context(module, parallel_context)
        self.memory_computation_balance = memory_computation_balance
        self.num_micro_batches = num_micro_batches
        self.pp_size = pc.get_world_size(ParallelMode.PIPELINE)
        self.stage = pc.get_local_rank(ParallelMode.PIPELINE)
        self.units: List[PipeUnit] = []
        self.my_units: List[PipeUnit] = []
        self._shared: List[nn.Parameter] = []
        self._meta_cache: Dict[str, tuple] = {}
        self.partition: List[range] = []
        self._tree = None  # set when the stages come from cutting the module tree
        self._grad_group = None  # second communicator over the pipeline ranks, for the backward direction
        add_wrapper(module, ParallelMode.PIPELINE, self)

    # ------------------------------------------------------------ parallelize
    def _get_units(self) -> List[PipeUnit]:
        if hasattr(self.module, "pipeline_units"):
            return self.module.pipeline_units()
        if isinstance(self.module, nn.Sequential):
            return sequential_units(self.module)
        # any other model: cut its module tree (embeddings / list of blocks / head), see tree_stage.py
        from .tree_stage import TreeStage

        self._tree = TreeStage(self.module)
        return self._tree.units()

    def _make_grad_group(self):
        """One more process group per pipeline group (collective over the whole job: every rank walks every list)."""
        pc = self.parallel_context
        if self.pp_size == 1 or not dist.is_initialized():
            return
        mine = sorted(pc.get_ranks_in_group(ParallelMode.PIPELINE))
        every = [None] * dist.get_world_size()
        dist.all_gather_object(every, mine)
        for ranks in sorted({tuple(r) for r in every}):
            g = dist.new_group(list(ranks))
            if tuple(mine) == ranks:
                self._grad_group = g

    @torch.no_grad()
    def parallelize(self):
        self._make_grad_group()
        self.units = self._get_units()
        self.partition = ModelPartitioner(self.units, self.pp_size, self.memory_computation_balance).partition()
        mine = self.partition[self.stage]
        self.my_units = [self.units[i] for i in mine]
        owner: Dict[int, set] = {}
        for s, r in enumerate(self.partition):
            for i in r:
                for p in self.units[i].parameters():
                    owner.setdefault(id(p), set()).add(s)
        keep = {id(p) for u in self.my_units for p in u.parameters()}
        for p in self.module.parameters():
            stages = owner.get(id(p), set())
            p.oslo_pipeline_stages = sorted(stages)
            if id(p) in keep:
                if len(stages) > 1:
                    self._shared.append(p)
            else:
                p.data = torch.empty(0, dtype=p.dtype, device=p.device)  # not ours: release the storage
                p.requires_grad_(False)
                p.oslo_pipeline_released = True
        if self._tree is not None:
            self._tree.install(mine, len(self.units), self.stage, self.pp_size)

    # ---------------------------------------------------------------- helpers
    def _split_kwargs(self, kwargs) -> List[dict]:
        m = self.num_micro_batches
        out = [dict() for _ in range(m)]
        for k, v in kwargs.items():
            if torch.is_tensor(v) and k in BATCH_DIMENSIONS_PP:
                dim = BATCH_DIMENSIONS_PP[k]
                if v.shape[dim] % m:
                    raise ValueError(f"batch dim of {k} ({v.shape[dim]}) is not divisible by num_micro_batches={m}")
                for i, c in enumerate(v.chunk(m, dim=dim)):
                    out[i][k] = c
            else:
                for i in range(m):
                    out[i][k] = v
        return out

    def _p2p_group(self, tag: str):
        if tag == "grad" and self._grad_group is not None:
            return self._grad_group
        return self.parallel_context.get_group(ParallelMode.PIPELINE)

    def _send(self, t: torch.Tensor, dst: int, tag: str):
        pc = self.parallel_context
        group = self._p2p_group(tag)
        t = t.contiguous()
        key = ("send", tag)  # shape / dtype travel once per direction and tag, then only payloads
        if self._meta_cache.get(key) != (tuple(t.shape), t.dtype):
            if key in self._meta_cache:
                raise RuntimeError("pipeline boundary tensors must keep their shape between micro-batches")
            P2P().send((tuple(t.shape), t.dtype), pc.get_global_rank(), dst, pc, ParallelMode.PIPELINE)
            self._meta_cache[key] = (tuple(t.shape), t.dtype)
        return dist.isend(t, dst=dst, group=group)

    def _post_recv(self, src: int, tag: str):
        """Post a non-blocking receive; returns ``(work, tensor)``.  The first receive of a tag learns shape and dtype
        from the sender (one object message), later ones reuse them."""
        pc = self.parallel_context
        key = ("recv", tag)
        if key not in self._meta_cache:
            self._meta_cache[key] = P2P().recv(src, pc.get_global_rank(), pc, ParallelMode.PIPELINE)
        shape, dtype = self._meta_cache[key]
        t = torch.empty(shape, dtype=dtype, device=pc.device)
        return dist.irecv(t, src=src, group=self._p2p_group(tag)), t

    def _recv(self, src: int, tag: str) -> torch.Tensor:
        work, t = self._post_recv(src, tag)
        work.wait()
        return t

    def _run_stage(self, state: dict) -> dict:
        if self._tree is not None:
            return self._tree.run(state)
        for u in self.my_units:
            state = u.fn(state)
        return state

    # ---------------------------------------------------------------- forward
    def forward(self, *args, **kwargs):
        if args:
            raise TypeError("pipeline-parallel models take keyword arguments only")
        return self._generator(kwargs)

    def _generator(self, kwargs):
        pc = self.parallel_context
        P, s, M = self.pp_size, self.stage, self.num_micro_batches
        first, last = s == 0, s == P - 1
        prev_rank = pc.get_prev_global_rank(ParallelMode.PIPELINE)
        next_rank = pc.get_next_global_rank(ParallelMode.PIPELINE)
        micro = self._split_kwargs(kwargs)
        if pc.tensor_parallel_size > 1 and pc.tensor_parallel_mode != ParallelMode.TENSOR_1D:
            # the stage functions bypass TensorParallel.forward, so the N-D input split happens here, per micro-batch
            from oslo_b200.parallel.tensor_parallel._wrapper_nd import scatter_batch_inputs

            micro = [scatter_batch_inputs(self.module, (), kw, pc)[1] for kw in micro]
        warmup = min(P - 1 - s, M)
        inputs: Dict[int, Optional[torch.Tensor]] = {}
        outputs: Dict[int, torch.Tensor] = {}
        pending = []
        self._meta_cache = {}  # shapes may change between calls (last partial batch, eval): re-announce them

        posted = {}  # micro-batch index -> (work, tensor) of an activation receive already in flight

        def forward_mb(i):
            state = dict(micro[i])
            if not first:
                work, h = posted.pop(i) if i in posted else self._post_recv(prev_rank, "act")
                work.wait()
                if i + 1 < M:
                    posted[i + 1] = self._post_recv(prev_rank, "act")  # runs under this micro-batch's compute
                h.requires_grad_(torch.is_grad_enabled() and h.is_floating_point())
                inputs[i] = h
                state["hidden"] = h
            state = self._run_stage(state)
            if last:
                loss = state.get("loss")
                if loss is not None:
                    loss = loss / M
                return PipelineOutput(loss=loss, logits=state.get("logits"))
            outputs[i] = state["hidden"]
            pending.append(self._send(state["hidden"].detach(), next_rank, "act"))
            return PipelineOutput(loss=_RemoteLoss())

        def backward_mb(j):
            if not last:
                g = self._recv(next_rank, "grad")
                torch.autograd.backward(outputs.pop(j), g)
            if not first:
                h = inputs.pop(j)
                if h.grad is not None:
                    pending.append(self._send(h.grad, prev_rank, "grad"))

        grad_mode = torch.is_grad_enabled()
        nf = nb = 0
        for _ in range(warmup):
            yield nf, forward_mb(nf)
            nf += 1
        while nf < M:
            out = forward_mb(nf)
            yield nf, out  # on the last stage the caller runs out.loss.backward() here
            nf += 1
            if grad_mode:
                backward_mb(nb)
                nb += 1
        while grad_mode and nb < M:
            backward_mb(nb)
            nb += 1
        for w in pending:
            w.wait()
        if grad_mode:
            self._sync_shared_grads()

    def _sync_shared_grads(self):
        """Sum gradients of parameters that live on several stages (tied embeddings)."""
        pc = self.parallel_context
        if self.pp_size == 1:
            return
        group = pc.get_group(ParallelMode.PIPELINE)
        # every rank of the pipeline group walks the same list of shared parameters (by name order)
        names = sorted(n for n, p in self.module.named_parameters() if len(getattr(p, "oslo_pipeline_stages", [])) > 1)
        params = dict(self.module.named_parameters())
        shapes = getattr(self, "_shared_shapes", None)
        if shapes is None:
            local = {n: (tuple(params[n].shape), params[n].dtype) for n in names if not getattr(params[n], "oslo_pipeline_released", False)}
            gathered = [None] * self.pp_size
            dist.all_gather_object(gathered, local, group=pc.get_cpu_group(ParallelMode.PIPELINE))
            shapes = {}
            for d in gathered:
                shapes.update(d)
            self._shared_shapes = shapes
        for n in names:
            p = params[n]
            shape, dtype = shapes[n]
            if getattr(p, "oslo_pipeline_released", False) or p.grad is None:
                buf = torch.zeros(shape, dtype=dtype, device=pc.device)
                dist.all_reduce(buf, group=group)
            else:
                dist.all_reduce(p.grad, group=group)

    def train_step(self, **kwargs):
        """Run one whole batch (all micro-batches, forward and backward); returns the summed micro-batch loss on the
        last stage and ``None`` elsewhere."""
        total = None
        for _, out in self(**kwargs):
            if not isinstance(out.loss, _RemoteLoss) and out.loss is not None:
                out.loss.backward()
                total = out.loss.detach() if total is None else total + out.loss.detach()
        return total

    # ------------------------------------------------------------ checkpoints
    def merge_state_dict_hook(self, state: dict) -> dict:
        """Fill in the tensors other stages own (collective over the PIPELINE group)."""
        pc = self.parallel_context
        if self.pp_size == 1:
            return state
        cpu_group = pc.get_cpu_group(ParallelMode.PIPELINE)
        params = dict(self.module.named_parameters())
        mine = {k: v for k, v in state.items() if not getattr(params.get(k), "oslo_pipeline_released", False)}
        gathered = [None] * self.pp_size
        dist.all_gather_object(gathered, mine, group=cpu_group)
        out = {}
        for d in gathered:
            for k, v in d.items():
                out.setdefault(k, v)
        return {k: out[k] for k in state if k in out}

    @torch.no_grad()
    def deparallelize(self):
        """Give every stage the full model again."""
        merged = self.merge_state_dict_hook({k: v.detach().cpu() for k, v in self.module.state_dict().items()})
        params = dict(self.module.named_parameters())
        for k, p in params.items():
            if getattr(p, "oslo_pipeline_released", False) and k in merged:
                p.data = merged[k].to(self.parallel_context.device)
                p.requires_grad_(True)
                p.oslo_pipeline_released = False
        if self._tree is not None:
            self._tree.uninstall()
