"""``ZeroRedundancyOptimizer``: ZeRO stage 1 / 2 with EVEN flat shards.

Design (differs from the reference on purpose): every (param group, dtype) is one flat buffer padded to a
multiple of the data-parallel size; rank ``r`` owns elements ``[r*S, (r+1)*S)`` of every bucket, keeps an fp32
master copy and the inner optimizer's state for that slice only.  One step is

    reduce-scatter(flat grads)  ->  inner optimizer on the fp32 master shard  ->  all-gather(flat params)

so communication is two bandwidth-optimal collectives regardless of how many tensors the model has.  The
reference assigns whole parameters to ranks (greedy by size, oslo/torch/nn/parallel/data_parallel/zero/optim/
optim.py:237-262), reduces bucket by bucket and re-broadcasts every owner's parameters one by one (:620-634).
On CUDA with the symmetric-memory runtime the three phases run as ONE kernel that pulls peers' gradient
slices over NVLink, applies AdamW and pushes the new parameters back (``csrc/zero_sm100a.cu``).

Buckets are reduced as soon as their gradients are complete when ``overlap_communication`` is set.
Parity: oslo/torch/nn/parallel/data_parallel/zero/optim/optim.py:138-666.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from oslo_b200.distributed import ParallelMode

from .._flat import FlatBuffer


class _Group:
    """One flat buffer (a dtype of a param group) and this rank's shard of it."""

    def __init__(self, flat: FlatBuffer, world: int, rank: int, bucket_elems: int, master_device):
        self.flat = flat
        self.world, self.rank = world, rank
        self.buckets = flat.bucket_ranges(bucket_elems, multiple=world)
        self.shard_ranges = []  # (flat_start, flat_end) owned by this rank, one per bucket
        for s, e in self.buckets:
            per = (e - s) // world
            self.shard_ranges.append((s + rank * per, s + (rank + 1) * per))
        self.shard_numel = sum(e - s for s, e in self.shard_ranges)
        self.master = torch.nn.Parameter(self._gather_shard(flat.param).float().to(master_device))
        self.master.grad = torch.zeros_like(self.master)
        self.pending = [0] * len(self.buckets)
        self.works = [None] * len(self.buckets)
        self.bucket_slots = [flat.slots_in(s, e) for s, e in self.buckets]

    def _gather_shard(self, buf: torch.Tensor) -> torch.Tensor:
        return torch.cat([buf[s:e] for s, e in self.shard_ranges])


class ZeroRedundancyOptimizer:
    def __init__(self, optimizer: torch.optim.Optimizer, parallel_context=None, clip_grad_norm: float = 0.0,
                 reduce_bucket_size: int = 64 * 1024 * 1024, communication_dtype: Optional[torch.dtype] = None,
                 overlap_communication: bool = False, partition_grad: bool = False, cpu_offload: bool = False,
                 forced_dtype: Optional[torch.dtype] = None, initial_scale: float = 1.0, growth_interval: int = 1000,
                 data_parallel_mode: ParallelMode = ParallelMode.DATA, fused: Optional[bool] = None):
        from oslo_b200.distributed import ParallelContext

        self.optim = optimizer
        self.pc = parallel_context or ParallelContext.get_context()
        self.mode = data_parallel_mode
        self.world = self.pc.get_world_size(self.mode)
        self.rank = self.pc.get_local_rank(self.mode)
        self.group = self.pc.get_group(self.mode)
        self.clip_grad_norm = clip_grad_norm
        self.partition_grad = partition_grad
        self.overlap = overlap_communication
        self.comm_dtype = communication_dtype
        self.cpu_offload = cpu_offload
        self.loss_scale = float(initial_scale)
        self.growth_interval, self._good_steps = growth_interval, 0
        self._groups: List[List[_Group]] = []
        self._callback_queued = False
        # fused path: flat buffers in symmetric memory and the whole step as one peer-memory kernel
        if fused is None:
            from oslo_b200.distributed import symm

            fused = symm.small_ops_enabled()
        inner_ok = type(optimizer).__name__ in ("Adam", "AdamW", "FusedAdam")
        self.fused = bool(fused and self.pc.use_cuda and self.world > 1 and self.world <= 8 and inner_ok and not cpu_offload)
        self._fused_state = {}
        self._param_to_bucket: Dict[int, tuple] = {}
        for pg in self.optim.param_groups:
            params = [p for p in pg["params"] if p.requires_grad]
            if forced_dtype is not None:
                for p in params:
                    p.data = p.data.to(forced_dtype)
            by_dtype: Dict[tuple, list] = {}
            for p in params:
                by_dtype.setdefault((p.dtype, p.device), []).append(p)
            groups = []
            for (dtype, device), ps in by_dtype.items():
                use_fused = self.fused and dtype in (torch.bfloat16, torch.float16)
                if use_fused:
                    from oslo_b200.distributed import symm

                    numel = FlatBuffer.layout_numel(ps, self.world * 128)
                    nbytes = numel * 2
                    sbuf = symm.SymmetricBuffer(self.pc, self.mode, 2 * nbytes)
                    flat = FlatBuffer(ps, pad_to=self.world * 128, with_grads=True, flatten_params=True,
                                      param_storage=sbuf.payload(0, nbytes, dtype), grad_storage=sbuf.payload(nbytes, nbytes, dtype))
                    reduce_bucket_size = numel  # one bucket: this rank's shard is one contiguous range
                    flat.symm, flat.symm_nbytes = sbuf, nbytes
                else:
                    flat = FlatBuffer(ps, pad_to=self.world * 128, with_grads=True, flatten_params=True)
                master_dev = torch.device("cpu") if cpu_offload else device
                g = _Group(flat, self.world, self.rank, reduce_bucket_size, master_dev)
                groups.append(g)
                for bi, slots in enumerate(g.bucket_slots):
                    for s in slots:
                        self._param_to_bucket.setdefault(id(s.param), []).append((g, bi))
                if self.overlap:
                    for p in ps:
                        p.register_post_accumulate_grad_hook(self._hook)
            self._groups.append(groups)
            pg["params"] = [g.master for g in groups]
        self.optim.state.clear()
        self._reset_pending()

    # ------------------------------------------------------------- plumbing
    @property
    def param_groups(self):
        return self.optim.param_groups

    @property
    def state(self):
        return self.optim.state

    def state_dict(self):
        """Inner optimizer state of THIS rank's shard (as the reference: no consolidation)."""
        return self.optim.state_dict()

    def load_state_dict(self, sd):
        self.optim.load_state_dict(sd)

    def _all_groups(self):
        for groups in self._groups:
            yield from groups

    def _reset_pending(self):
        for g in self._all_groups():
            g.pending = [len(s) for s in g.bucket_slots]
            g.works = [None] * len(g.buckets)

    def zero_grad(self, set_to_none: bool = True):
        for g in self._all_groups():
            g.flat.zero_grad()

    def backward(self, loss, retain_graph: bool = False):
        (loss * self.loss_scale).backward(retain_graph=retain_graph)

    # -------------------------------------------------- gradient reduction
    def _hook(self, p):
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._backward_done)
        for g, bi in self._param_to_bucket.get(id(p), ()):
            g.pending[bi] -= 1
            if g.pending[bi] == 0:
                self._reduce_bucket(g, bi, async_op=True)

    def _backward_done(self):
        self._callback_queued = False

    def _reduce_bucket(self, g: _Group, bi: int, async_op: bool):
        if self.world == 1 or g.works[bi] is not None:
            return
        s, e = g.buckets[bi]
        view = g.flat.grad[s:e]
        for slot in g.bucket_slots[bi]:  # gradients re-pointed by the user are copied back into the flat buffer
            gr = slot.param.grad
            if gr is not None and gr.data_ptr() != g.flat.grad[slot.offset : slot.offset + slot.numel].data_ptr():
                g.flat.grad[slot.offset : slot.offset + slot.numel].copy_(gr.reshape(-1))
        buf = view if self.comm_dtype in (None, view.dtype) else view.to(self.comm_dtype)
        buf.div_(self.world)
        if self.partition_grad and dist.get_backend(self.group) != "gloo":
            per = (e - s) // self.world
            out = buf[self.rank * per : (self.rank + 1) * per]
            work = dist.reduce_scatter_tensor(out, buf, group=self.group, async_op=async_op)
        else:
            work = dist.all_reduce(buf, group=self.group, async_op=async_op)
        g.works[bi] = (work, buf, view)

    def _finish_reduction(self):
        for g in self._all_groups():
            for bi in range(len(g.buckets)):
                if g.works[bi] is None:
                    self._reduce_bucket(g, bi, async_op=False)
                if g.works[bi] is not None:
                    work, buf, view = g.works[bi]
                    if work is not None:
                        work.wait()
                    if buf is not view:
                        view.copy_(buf)

    # ----------------------------------------------------------------- step
    def _grad_shards_to_master(self):
        for g in self._all_groups():
            shard = g._gather_shard(g.flat.grad)
            g.master.grad.copy_(shard.to(g.master.device, non_blocking=True).float())

    def _global_norm_and_overflow(self):
        sq = torch.zeros(1, dtype=torch.float32, device=self.pc.device)
        for g in self._all_groups():
            sq += g.master.grad.float().pow(2).sum().to(sq.device)
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        pc = self.pc
        # tensor-parallel shards hold disjoint parameter slices: their squared norms add up
        if pc.is_initialized(ParallelMode.TENSOR) and pc.get_world_size(ParallelMode.TENSOR) > 1:
            dist.all_reduce(sq, group=pc.get_group(ParallelMode.TENSOR))
        if pc.is_initialized(ParallelMode.PIPELINE) and pc.get_world_size(ParallelMode.PIPELINE) > 1:
            dist.all_reduce(sq, group=pc.get_group(ParallelMode.PIPELINE))
        norm = sq.sqrt().item()
        return norm, not math.isfinite(norm)

    def _fused_step_group(self, g: _Group, pg: dict, step_no: int):
        """reduce-scatter + AdamW + all-gather for one flat buffer as one kernel (``csrc/zero_sm100a.cu``)."""
        import ctypes

        from oslo_b200.ops import _lib

        flat, sbuf = g.flat, g.flat.symm
        st = self._fused_state.get(id(g))
        if st is None:
            st = self._fused_state[id(g)] = dict(m=torch.zeros_like(g.master.data), v=torch.zeros_like(g.master.data))
        (s0, e0) = g.shard_ranges[0]
        b1, b2 = pg.get("betas", (0.9, 0.999))
        lib = _lib.cuda_lib()
        grads, params = sbuf.peer_array(flat.symm_nbytes), sbuf.peer_array(0)
        common = [ctypes.c_longlong(s0), ctypes.c_longlong(e0 - s0), ctypes.c_int(self.world),
                  ctypes.c_int(1 if flat.dtype == torch.bfloat16 else 0), ctypes.c_float(pg["lr"]), ctypes.c_float(b1),
                  ctypes.c_float(b2), ctypes.c_float(pg.get("eps", 1e-8)), ctypes.c_float(pg.get("weight_decay", 0.0)),
                  ctypes.c_float(1 - b1**step_no), ctypes.c_float(1 - b2**step_no),
                  ctypes.c_float(1.0 / (self.world * self.loss_scale)),
                  ctypes.c_int(0 if type(self.optim).__name__ == "Adam" else 1)]
        sbuf.barrier()  # every rank's gradients are final
        coef = None
        if self.clip_grad_norm > 0:
            sq = torch.zeros(1, dtype=torch.float32, device=flat.device)
            rc = lib.oslo_zero_step(grads, params, _lib.ptr(g.master.data), _lib.ptr(st["m"]), _lib.ptr(st["v"]), *common,
                                    ctypes.c_int(0), None, _lib.ptr(sq), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
            if rc:
                raise RuntimeError(f"oslo_zero_step (norm) failed ({rc})")
            dist.all_reduce(sq, group=self.group)
            coef = (self.clip_grad_norm / (sq.sqrt() + 1e-6)).clamp(max=1.0)
            self.last_grad_norm = sq.sqrt()
        rc = lib.oslo_zero_step(grads, params, _lib.ptr(g.master.data), _lib.ptr(st["m"]), _lib.ptr(st["v"]), *common,
                                ctypes.c_int(1), _lib.ptr(coef), None, ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_zero_step failed ({rc})")
        sbuf.barrier()  # every rank's parameters have landed everywhere

    @torch.no_grad()
    def step(self, closure=None):
        if self.fused and all(hasattr(g.flat, "symm") for g in self._all_groups()):
            self._step_count = getattr(self, "_step_count", 0) + 1
            for groups, pg in zip(self._groups, self.optim.param_groups):
                for g in groups:
                    self._fused_step_group(g, pg, self._step_count)
            self._reset_pending()
            return None
        self._finish_reduction()
        self._grad_shards_to_master()
        norm, overflow = self._global_norm_and_overflow()
        if overflow:
            # skip the update, shrink the loss scale (dynamic scaling for fp16)
            self.loss_scale = max(self.loss_scale / 2.0, 1.0)
            self._good_steps = 0
            self.zero_grad()
            self._reset_pending()
            return None
        unscale = 1.0 / self.loss_scale
        norm *= unscale
        coef = unscale
        if self.clip_grad_norm > 0 and norm > self.clip_grad_norm:
            coef *= self.clip_grad_norm / (norm + 1e-6)
        if coef != 1.0:
            for g in self._all_groups():
                g.master.grad.mul_(coef)
        self.optim.step()
        self._good_steps += 1
        if self.loss_scale > 1.0 and self._good_steps % self.growth_interval == 0:
            self.loss_scale *= 2.0
        for g in self._all_groups():
            new = g.master.data.to(g.flat.param.device, non_blocking=True).to(g.flat.dtype)
            off = 0
            for s, e in g.shard_ranges:
                g.flat.param[s:e].copy_(new[off : off + (e - s)])
                off += e - s
            if self.world > 1:
                for (s, e), (ss, se) in zip(g.buckets, g.shard_ranges):
                    dist.all_gather_into_tensor(g.flat.param[s:e], g.flat.param[ss:se].clone(), group=self.group)
        self._reset_pending()
        self.last_grad_norm = norm
        return None
