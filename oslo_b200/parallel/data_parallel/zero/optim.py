"""``ZeroRedundancyOptimizer``: ZeRO stage 1 / 2 with EVEN flat shards.

Design (differs from the reference on purpose): every (param group, dtype) is one flat buffer padded to a
multiple of the data-parallel size; rank ``r`` owns elements ``[r*S, (r+1)*S)`` of every bucket, keeps an fp32
master copy and the inner optimizer's state for that slice only.  One step is

    reduce-scatter(flat grads)  ->  inner optimizer on the fp32 master shard  ->  all-gather(flat params)

so communication is two bandwidth-optimal collectives regardless of how many tensors the model has.  The
reference assigns whole parameters to ranks (greedy by size, oslo/torch/nn/parallel/data_parallel/zero/optim/
optim.py:237-262), reduces bucket by bucket and re-broadcasts every owner's parameters one by one (:620-634).
On CUDA with the symmetric-memory runtime the three phases run as ONE kernel per bucket that pulls peers' gradient
slices over NVLink, applies AdamW and pushes the new parameters back (``csrc/zero_sm100a.cu``).

Buckets are reduced as soon as their gradients are complete when ``overlap_communication`` is set.  On the fused
path that means: a bucket's kernel is launched on a side stream from the gradient hook of the bucket's last
parameter, behind a device barrier over the data-parallel group, so the NVLink traffic of the reduce-scatter (and,
when no clipping or loss scaling is asked for, the update and the parameter push as well) runs under the rest of
backward.  With clipping, the kernel keeps the reduced fp32 shard and its squared norm instead (one pull only); the
update from that shard runs in ``step()`` once the global norm is known.

Gradient accumulation: run every backward but the last one of a step inside ``no_sync()``; a gradient that arrives for
a bucket that was already reduced in this step raises instead of being silently dropped.
Parity: oslo/torch/nn/parallel/data_parallel/zero/optim/optim.py:138-666.
"""
from __future__ import annotations

import contextlib
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
        self.buckets = flat.bucket_ranges(bucket_elems, multiple=world * 128)
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
        # offset of every bucket's shard inside the master / moment tensors
        self.master_offsets, off = [], 0
        for s, e in self.shard_ranges:
            self.master_offsets.append(off)
            off += e - s
        self.launched = [False] * len(self.buckets)  # fused path: this bucket's kernel is already in flight

    def resync_master(self):
        """Re-copy the fp32 master shard from the (possibly reloaded) low-precision parameters."""
        self.master.data.copy_(self._gather_shard(self.flat.param).float().to(self.master.device))

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
        self._sync = True  # False inside no_sync(): gradients accumulate locally, nothing is reduced
        self._step_count = 0
        self.last_grad_norm = None
        # fused path: flat buffers in symmetric memory and the whole step as one peer-memory kernel per bucket
        if fused is None:
            from oslo_b200.distributed import symm

            fused = symm.small_ops_enabled()
        inner_ok = type(optimizer).__name__ in ("Adam", "AdamW", "FusedAdam")
        self.fused = bool(fused and self.pc.use_cuda and self.world > 1 and self.world <= 8 and inner_ok and not cpu_offload)
        self._fused_state = {}
        self._comm_stream = None
        self._sumsq = None
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
        self._all_fused = self.fused and all(hasattr(g.flat, "symm") for g in self._all_groups())
        self._reset_pending()

    # ------------------------------------------------------------- plumbing
    @property
    def param_groups(self):
        return self.optim.param_groups

    @property
    def state(self):
        return self.optim.state

    def state_dict(self):
        """State of THIS rank's shard (as the reference: no consolidation): the inner optimizer's state, the fp32
        master shards, the moments of the fused path, the step count and the loss scale."""
        fused = []
        for g in self._all_groups():
            st = self._fused_state.get(id(g))
            fused.append(None if st is None else {"m": st["m"].detach().cpu(), "v": st["v"].detach().cpu()})
        return {
            "zero_format": 2,
            "inner": self.optim.state_dict(),
            "masters": [g.master.data.detach().cpu() for g in self._all_groups()],
            "fused_moments": fused,
            "step_count": self._step_count,
            "loss_scale": self.loss_scale,
            "good_steps": self._good_steps,
        }

    def load_state_dict(self, sd):
        if "zero_format" not in sd:  # an inner-optimizer state dict only
            self.optim.load_state_dict(sd)
            self.resync_master()
            return
        self.optim.load_state_dict(sd["inner"])
        groups = list(self._all_groups())
        if len(sd["masters"]) != len(groups):
            raise ValueError("checkpoint has a different number of flat groups than this optimizer")
        for g, m, fm in zip(groups, sd["masters"], sd["fused_moments"]):
            if m.numel() != g.master.numel():
                raise ValueError("master shard size mismatch: the checkpoint was written with another data-parallel size")
            g.master.data.copy_(m.to(g.master.device))
            if fm is not None:
                self._fused_state[id(g)] = dict(m=fm["m"].to(g.master.device).clone(), v=fm["v"].to(g.master.device).clone())
        self._step_count = int(sd.get("step_count", 0))
        self.loss_scale = float(sd.get("loss_scale", self.loss_scale))
        self._good_steps = int(sd.get("good_steps", 0))

    def resync_master(self):
        """Refresh every fp32 master shard from the model's current parameters.  Call after loading weights into a model
        that is already wrapped (``load_state_dict`` / ``from_parallelized``): otherwise the next ``step()`` writes the
        stale masters over the loaded weights."""
        for g in self._all_groups():
            g.resync_master()

    def _all_groups(self):
        for groups in self._groups:
            yield from groups

    def _reset_pending(self):
        for g in self._all_groups():
            g.pending = [len(s) for s in g.bucket_slots]
            g.works = [None] * len(g.buckets)
            g.launched = [False] * len(g.buckets)

    def zero_grad(self, set_to_none: bool = True):
        for g in self._all_groups():
            g.flat.zero_grad()

    def backward(self, loss, retain_graph: bool = False):
        (loss * self.loss_scale).backward(retain_graph=retain_graph)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate gradients locally (gradient accumulation, pipeline
        micro-batches); the reduction is issued by the first backward outside of it, or by ``step()``."""
        prev, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = prev

    # -------------------------------------------------- gradient reduction
    def _hook(self, p):
        if not self._sync:
            return
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._backward_done)
        for g, bi in self._param_to_bucket.get(id(p), ()):
            if g.works[bi] is not None or g.launched[bi]:
                raise RuntimeError(
                    "ZeroRedundancyOptimizer(overlap_communication=True): a gradient arrived for a bucket that was already "
                    "reduced in this step. Run every backward of a step but the last one inside `optimizer.no_sync()`.")
            g.pending[bi] -= 1
            if g.pending[bi] == 0:
                if self._all_fused:
                    self._launch_fused_bucket(g, bi, overlapped=True)
                else:
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

    def _reduce_norm_sq(self, sq: torch.Tensor) -> torch.Tensor:
        """Sum a squared gradient norm over the data-parallel shards and over the tensor- and pipeline-parallel ranks
        (which hold disjoint parameter slices), so every rank of the job clips with the same coefficient."""
        pc = self.pc
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        if pc.is_initialized(ParallelMode.TENSOR) and pc.get_world_size(ParallelMode.TENSOR) > 1:
            dist.all_reduce(sq, group=pc.get_group(ParallelMode.TENSOR))
        if pc.is_initialized(ParallelMode.PIPELINE) and pc.get_world_size(ParallelMode.PIPELINE) > 1:
            dist.all_reduce(sq, group=pc.get_group(ParallelMode.PIPELINE))
        return sq

    def _global_norm_and_overflow(self):
        sq = torch.zeros(1, dtype=torch.float32, device=self.pc.device)
        for g in self._all_groups():
            sq += g.master.grad.float().pow(2).sum().to(sq.device)
        norm = self._reduce_norm_sq(sq).sqrt().item()
        return norm, not math.isfinite(norm)

    # ----------------------------------------------------------- fused path
    def _two_phase(self) -> bool:
        """Clipping and loss scaling need the global norm before any update: buckets are reduced first (one pull, fp32
        shard kept) and updated afterwards.  Otherwise a bucket is reduced, updated and pushed by a single kernel."""
        return self.clip_grad_norm > 0 or self.loss_scale != 1.0

    def _fused_args(self, g: _Group, pg: dict):
        import ctypes

        flat = g.flat
        b1, b2 = pg.get("betas", (0.9, 0.999))
        n = max(self._step_count, 1)
        return [ctypes.c_int(self.world), ctypes.c_int(1 if flat.dtype == torch.bfloat16 else 0), ctypes.c_float(pg["lr"]),
                ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(pg.get("eps", 1e-8)),
                ctypes.c_float(pg.get("weight_decay", 0.0)), ctypes.c_float(1 - b1**n), ctypes.c_float(1 - b2**n),
                ctypes.c_float(1.0 / (self.world * self.loss_scale)),
                ctypes.c_int(0 if type(self.optim).__name__ == "Adam" else 1)]

    def _moments(self, g: _Group):
        st = self._fused_state.get(id(g))
        if st is None:
            st = self._fused_state[id(g)] = dict(m=torch.zeros_like(g.master.data), v=torch.zeros_like(g.master.data))
        return st

    def _pg_of(self, g: _Group) -> dict:
        for groups, pg in zip(self._groups, self.optim.param_groups):
            if any(x is g for x in groups):
                return pg
        raise KeyError("group not registered")

    def _begin_fused_step(self):
        """First fused launch of a step: advance the step count (bias corrections) and clear the norm accumulator."""
        if getattr(self, "_fused_step_open", False):
            return
        self._fused_step_open = True
        self._step_count += 1
        dev = self.pc.device
        if self._sumsq is None:
            self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=dev)
        self._sumsq.zero_()

    def _launch_fused_bucket(self, g: _Group, bi: int, overlapped: bool):
        """Barrier over the data-parallel group (this bucket's gradients are final everywhere), then the bucket's kernel.
        ``overlapped``: issue both on the side stream so they run under the rest of backward."""
        import ctypes

        from oslo_b200.ops import _lib

        if g.launched[bi]:
            return
        self._begin_fused_step()
        g.launched[bi] = True
        flat, sbuf = g.flat, g.flat.symm
        st = self._moments(g)
        s0, e0 = g.shard_ranges[bi]
        moff = g.master_offsets[bi]
        two_phase = self._two_phase()
        lib = _lib.cuda_lib()
        grads, params = sbuf.peer_array(flat.symm_nbytes), sbuf.peer_array(0)
        stream = self._comm_stream if overlapped else torch.cuda.current_stream()
        if overlapped:
            stream.wait_stream(torch.cuda.current_stream())
        from oslo_b200.utils.nvtx import annotate

        with torch.cuda.stream(stream), annotate("oslo.zero_bucket"):
            sbuf.barrier()
            rc = lib.oslo_zero_step(
                grads, params, _lib.ptr(g.master.data[moff:]), _lib.ptr(st["m"][moff:]), _lib.ptr(st["v"][moff:]),
                ctypes.c_longlong(s0), ctypes.c_longlong(e0 - s0), *self._fused_args(g, self._pg_of(g)),
                ctypes.c_int(2 if two_phase else 1), None, _lib.ptr(self._sumsq) if two_phase else None,
                ctypes.c_int(_lib.num_sms()), _lib.stream_ptr(), _lib.ptr(g.master.grad[moff:]) if two_phase else None)
        if rc:
            raise RuntimeError(f"oslo_zero_step failed ({rc})")

    def _fused_step(self):
        import ctypes

        from oslo_b200.ops import _lib

        for g in self._all_groups():
            for bi in range(len(g.buckets)):
                self._launch_fused_bucket(g, bi, overlapped=False)
        cur = torch.cuda.current_stream()
        if self._comm_stream is not None:
            cur.wait_stream(self._comm_stream)
        skipped = False
        if self._two_phase():
            sq = self._reduce_norm_sq(self._sumsq)
            norm = sq.sqrt()
            self.last_grad_norm = norm
            coef = torch.ones_like(norm)
            if self.clip_grad_norm > 0:
                coef = (self.clip_grad_norm / (norm + 1e-6)).clamp(max=1.0)
            coef = torch.where(torch.isfinite(norm), coef, torch.full_like(coef, float("nan")))
            if self.loss_scale != 1.0:  # dynamic loss scaling needs the verdict on the host
                skipped = not bool(torch.isfinite(norm).item())
            lib = _lib.cuda_lib()
            for g in self._all_groups():
                flat, sbuf = g.flat, g.flat.symm
                st = self._moments(g)
                grads, params = sbuf.peer_array(flat.symm_nbytes), sbuf.peer_array(0)
                for bi, (s0, e0) in enumerate(g.shard_ranges):
                    moff = g.master_offsets[bi]
                    rc = lib.oslo_zero_step(
                        grads, params, _lib.ptr(g.master.data[moff:]), _lib.ptr(st["m"][moff:]), _lib.ptr(st["v"][moff:]),
                        ctypes.c_longlong(s0), ctypes.c_longlong(e0 - s0), *self._fused_args(g, self._pg_of(g)),
                        ctypes.c_int(3), _lib.ptr(coef), None, ctypes.c_int(_lib.num_sms()), _lib.stream_ptr(),
                        _lib.ptr(g.master.grad[moff:]))
                    if rc:
                        raise RuntimeError(f"oslo_zero_step (update) failed ({rc})")
        for g in self._all_groups():
            g.flat.symm.barrier()  # every rank's parameters have landed everywhere
        self._fused_step_open = False
        if skipped:
            self._step_count -= 1
            self.loss_scale = max(self.loss_scale / 2.0, 1.0)
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self.loss_scale > 1.0 and self._good_steps % self.growth_interval == 0:
                self.loss_scale *= 2.0
        self._reset_pending()

    @torch.no_grad()
    def step(self, closure=None):
        if self._all_fused:
            self._fused_step()
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
        self._step_count += 1
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
