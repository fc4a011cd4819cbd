"""Symmetric memory for a process group: one device allocation per rank, mapped into every peer (CUDA IPC).

``enable(parallel_context, mode, max_tokens, max_features)`` builds a :class:`SymmetricWorkspace` for the
group and registers it with :mod:`oslo_b200.ops.fused_collectives`, after which the sequence-parallel linears
run as single fused kernels (``csrc/fused_collectives_sm100a.cu``).

Workspace layout per rank (all offsets identical on every rank)::

    [ flags 4 KiB | gathered[0] | gathered[1] | slots[0] | slots[1] ]

* ``gathered[p]``  the all-gather result of calls with parity ``p`` (``T x F`` elements): rank ``s`` PUSHES its shard into
                   block ``s`` of this buffer on every rank (remote writes are posted, remote reads are latency-bound);
* ``slots[p]``     ``tp`` blocks of ``Tl x F``: block ``s`` receives rank ``s``'s partial rows of a reduce-scatter;
* flags           ``chunk_flag[tp * chunks]`` (a source has delivered that row chunk), ``rs_flag[..]``, ``barrier[tp]``,
                   all written by peers and holding call epochs.

Double buffering by call parity is what makes the scheme free of write-after-read races without a trailing
barrier: a rank can only be one call ahead of any peer, because each call needs data from every peer.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from oslo_b200.ops import _lib, fused_collectives

_FLAG_BYTES = 4096

#: use NVSwitch multicast (``multimem`` stores and in-switch reductions) in the fused kernels when the group's workspace can
#: be bound to a multicast object; OSLO_B200_MULTIMEM=0 keeps plain peer loads / stores (required for any test in which a
#: rank may leave while others still run: a rank that dies while bound to a multicast object faults its peers' links).
USE_MULTIMEM = __import__("os").environ.get("OSLO_B200_MULTIMEM", "1") == "1"


#: move the shards of the fused 1-D kernels with the copy engines (``cudaMemcpyAsync`` between peer mappings on side
#: streams, flags written the same way) instead of with copy CTAs / epilogue stores: the links then run at copy-engine
#: speed and every SM multiplies.  OSLO_B200_CE_TRANSPORT=0 keeps the in-kernel transports.
USE_CE_TRANSPORT = __import__("os").environ.get("OSLO_B200_CE_TRANSPORT", "0") == "1"


def _multicast_alloc(pc, mode, nbytes: int):
    """Allocate ``nbytes`` per rank through ``torch.distributed._symmetric_memory`` and rendezvous over the group.

    Returns ``(tensor, peer_pointers, multicast_pointer)`` or ``None`` when the allocation, the exchange of handles or the
    multicast binding is not available (the caller then uses its CUDA-IPC allocation).  Collective over the group: every
    rank must take the same branch, so the outcome is agreed on with an all-reduce."""
    ok, out = 1, None
    try:
        import torch.distributed._symmetric_memory as symm_mem

        group = pc.get_group(mode)
        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=pc.device)
        hdl = symm_mem.rendezvous(t, group)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        ptrs = [int(x) for x in hdl.buffer_ptrs]
        if mc == 0 or len(ptrs) != pc.get_world_size(mode):
            ok = 0
        else:
            out = (t, hdl, ptrs, mc)
    except Exception as e:  # noqa: BLE001 - any failure means "not available here"
        ok = 0
        out = None
        _multicast_alloc.last_error = repr(e)
    flag = torch.tensor([ok], dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pc.get_cpu_group(mode))
    return out if int(flag.item()) == 1 else None


_multicast_alloc.last_error = None


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__`` (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of a group, each rank's block mapped into all the others.

    ``local`` is a ``uint8`` tensor over this rank's block; ``peer_ptrs[r]`` the address of rank ``r``'s block in this
    process.  The first 1 KiB holds flags used by :meth:`barrier` (a bounded device-side barrier on the current
    stream); ``payload_offset`` is where user data starts.
    """

    payload_offset = 1024

    def __init__(self, pc, mode, nbytes: int):
        self.pc, self.mode = pc, mode
        self.world = pc.get_world_size(mode)
        self.rank = pc.get_local_rank(mode)
        if self.world > 8:
            raise ValueError("symmetric buffers support groups of up to 8 ranks")
        self.device = pc.device
        self.nbytes = (nbytes + self.payload_offset + 1023) // 1024 * 1024
        lib = _lib.cuda_lib()
        base = ctypes.c_void_p()
        rc = lib.oslo_symm_alloc(ctypes.c_ulonglong(self.nbytes), ctypes.byref(base))
        if rc:
            raise RuntimeError(f"symmetric allocation of {self.nbytes} bytes failed (cuda error {-rc})")
        self.base = base.value
        hbytes = lib.oslo_ipc_handle_bytes()
        handle = (ctypes.c_ubyte * hbytes)()
        rc = lib.oslo_ipc_get_handle(ctypes.c_void_p(self.base), handle)
        if rc:
            raise RuntimeError(f"cudaIpcGetMemHandle failed (cuda error {-rc})")
        gathered: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=pc.get_cpu_group(mode))
        self.peer_ptrs: List[int] = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                self.peer_ptrs.append(self.base)
                continue
            buf = (ctypes.c_ubyte * hbytes).from_buffer_copy(h)
            out = ctypes.c_void_p()
            rc = lib.oslo_ipc_open_handle(buf, ctypes.byref(out))
            if rc:
                raise RuntimeError(f"cudaIpcOpenMemHandle for peer {r} failed (cuda error {-rc})")
            self.peer_ptrs.append(out.value)
        self.local = torch.as_tensor(_RawCudaBuffer(self.base, self.nbytes), device=self.device)
        self.epoch = 0
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)  # what the kernels actually read
        dist.barrier(group=pc.get_cpu_group(mode))

    def payload(self, offset: int, nbytes: int, dtype, shape=None) -> torch.Tensor:
        t = self.local[self.payload_offset + offset : self.payload_offset + offset + nbytes].view(dtype)
        return t.view(shape) if shape is not None else t

    def peer_array(self, offset: int = 0):
        """ctypes array of every rank's address of ``payload + offset``."""
        return (ctypes.c_void_p * self.world)(*[b + self.payload_offset + offset for b in self.peer_ptrs])

    def barrier(self):
        self.epoch += 1
        self.epoch_dev.add_(1)  # a stream-ordered (and graph-capturable) increment
        flags = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        rc = _lib.cuda_lib().oslo_symm_barrier(flags, ctypes.c_void_p(self.base), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                               ctypes.c_int(self.epoch), _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr(),
                                               _lib.ptr(self.epoch_dev))
        if rc:
            raise RuntimeError(f"oslo_symm_barrier failed ({rc})")


_group_buffers = {}


def group_buffer(pc, mode, key: str, nbytes: int) -> "SymmetricBuffer":
    """A cached :class:`SymmetricBuffer` per (context, mode, key); grown (re-created) when a larger size is asked for.
    Collective over the group."""
    k = (id(pc), mode, key)
    buf = _group_buffers.get(k)
    if buf is None or buf.nbytes < nbytes + SymmetricBuffer.payload_offset:
        buf = _group_buffers[k] = SymmetricBuffer(pc, mode, nbytes)
    return buf


def rehome_parameter(pc, mode, param: torch.nn.Parameter) -> "SymmetricBuffer":
    """Move a parameter's storage into symmetric memory (its shard becomes readable by every rank of the group).
    The Parameter object is kept, so tied weights stay tied.  Collective over the group."""
    nbytes = param.numel() * param.element_size()
    buf = SymmetricBuffer(pc, mode, nbytes)
    view = buf.payload(0, nbytes, param.dtype, tuple(param.shape))
    view.copy_(param.data)
    param.data = view
    param.oslo_symm = buf
    return buf


def rehome_vocab_embeddings(model, pc, mode) -> int:
    """Put every ``VocabParallelEmbedding1D`` table of ``model`` into symmetric memory so its lookups read the owning
    rank directly; returns how many were moved."""
    from oslo_b200.nn.embedding import VocabParallelEmbedding1D

    n = 0
    for m in model.modules():
        if isinstance(m, VocabParallelEmbedding1D) and m.weight.is_cuda and not hasattr(m.weight, "oslo_symm"):
            if (m.weight.shape[1] * m.weight.element_size()) % 16 == 0:
                rehome_parameter(pc, mode, m.weight)
                n += 1
    return n


_fused_small_ops = False


def small_ops_enabled() -> bool:
    """True once :func:`enable` ran: the loss / embedding / optimizer paths may use peer memory too."""
    return _fused_small_ops


class SymmetricWorkspace:
    def __init__(self, pc, mode, max_tokens: int, max_features: int, dtype=torch.bfloat16, copy_ctas: int = 16,
                 multimem: bool = True, ce_transport: Optional[bool] = None):
        self.pc, self.mode = pc, mode
        self.tp = pc.get_world_size(mode)
        self.rank = pc.get_local_rank(mode)
        if self.tp > 8:
            raise ValueError("fused collectives support groups of up to 8 ranks")
        self.device = pc.device
        self.dtype = dtype
        self.copy_ctas = copy_ctas
        self.max_tokens, self.max_features = max_tokens, max_features
        esz = torch.empty((), dtype=dtype).element_size()
        if ce_transport is None:
            ce_transport = USE_CE_TRANSPORT
        self.in_bytes = (max_tokens * max_features * esz + 1023) // 1024 * 1024  # one gathered buffer
        self.slot_bytes = (max_tokens * max_features * esz + 1023) // 1024 * 1024
        self.total = _FLAG_BYTES + 2 * self.in_bytes + 2 * self.slot_bytes
        lib = _lib.cuda_lib()
        #: address of the whole workspace through the group's NVSwitch multicast object (0: not bound)
        self.mc_base = 0
        self._symm_keep = None
        # measured on the flagship step: multicast is ahead at eight ranks (47.5 vs 49.1 ms) and behind at four (63.8 vs 60.6)
        # and two, where a shard crosses the links once or thrice either way; OSLO_B200_MULTIMEM_MIN_RANKS moves the threshold
        min_ranks = int(__import__("os").environ.get("OSLO_B200_MULTIMEM_MIN_RANKS", "8"))
        mc = _multicast_alloc(pc, mode, self.total) if (USE_MULTIMEM and multimem and self.tp >= min_ranks) else None
        if mc is not None:
            tensor, hdl, ptrs, mc_ptr = mc
            tensor.zero_()
            torch.cuda.synchronize(self.device)
            self._symm_keep = (tensor, hdl)
            self.base = tensor.data_ptr()
            self.peer_base: List[int] = ptrs
            self.mc_base = mc_ptr
        else:
            base = ctypes.c_void_p()
            rc = lib.oslo_symm_alloc(ctypes.c_ulonglong(self.total), ctypes.byref(base))
            if rc:
                raise RuntimeError(f"symmetric allocation of {self.total} bytes failed (cuda error {-rc})")
            self.base = base.value
            hbytes = lib.oslo_ipc_handle_bytes()
            handle = (ctypes.c_ubyte * hbytes)()
            rc = lib.oslo_ipc_get_handle(ctypes.c_void_p(self.base), handle)
            if rc:
                raise RuntimeError(f"cudaIpcGetMemHandle failed (cuda error {-rc})")
            gathered: List[Optional[bytes]] = [None] * self.tp
            dist.all_gather_object(gathered, bytes(handle), group=pc.get_cpu_group(mode))
            self.peer_base = []
            for r, h in enumerate(gathered):
                if r == self.rank:
                    self.peer_base.append(self.base)
                    continue
                buf = (ctypes.c_ubyte * hbytes).from_buffer_copy(h)
                out = ctypes.c_void_p()
                rc = lib.oslo_ipc_open_handle(buf, ctypes.byref(out))
                if rc:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for peer {r} failed (cuda error {-rc})")
                self.peer_base.append(out.value)
        # local scratch counters (not shared): chunk_flag[64], chunk_arrive[64], tile_done[64]
        self.local = torch.zeros(256, dtype=torch.int32, device=self.device)
        self.epoch = 0
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)  # what the kernels actually read
        self.debug_times = None  # set to a uint64[8] device tensor to collect in-kernel time stamps
        if self._symm_keep is not None:
            self._local_bytes = self._symm_keep[0]
        else:
            self._local_bytes = torch.as_tensor(_RawCudaBuffer(self.base, self.total), device=self.device)
        # Copy-engine transport (see ``_ag_gemm_ce`` / ``_gemm_rs_ce``): every rank's workspace as a tensor in this process,
        # one stream per destination so the transfers to different peers run on different copy engines, two local staging
        # buffers for partial blocks on their way out.
        self.ce_transport = bool(ce_transport) and not self.mc_base
        self._peer_bytes = [self._local_bytes if r == self.rank else torch.as_tensor(_RawCudaBuffer(b, self.total), device=self.device)
                            for r, b in enumerate(self.peer_base)]
        self._ce_streams = [torch.cuda.Stream(device=self.device) for _ in range(self.tp)] if self.ce_transport else []
        self._stage = None
        self._stage_free = [None, None]
        dist.barrier(group=pc.get_cpu_group(mode))
        self.barrier()

    # ------------------------------------------------------------ addressing
    def _flag_ptrs(self, which: int):
        # which: 0 chunk_flag (all-gather), 1 rs_flag, 2 barrier ; each 64 ints apart
        return (ctypes.c_void_p * self.tp)(*[b + which * 256 for b in self.peer_base])

    def _gathered_ptrs(self, parity: int):
        off = _FLAG_BYTES + parity * self.in_bytes
        return (ctypes.c_void_p * self.tp)(*[b + off for b in self.peer_base])

    def _slot_ptrs(self, parity: int):
        off = _FLAG_BYTES + 2 * self.in_bytes + parity * self.slot_bytes
        return (ctypes.c_void_p * self.tp)(*[b + off for b in self.peer_base])

    def _mc_gathered(self, parity: int):
        return ctypes.c_void_p(self.mc_base + _FLAG_BYTES + parity * self.in_bytes) if self.mc_base else ctypes.c_void_p(0)

    def _mc_slots(self, parity: int):
        if not self.mc_base:
            return ctypes.c_void_p(0)
        return ctypes.c_void_p(self.mc_base + _FLAG_BYTES + 2 * self.in_bytes + parity * self.slot_bytes)

    def _local_gathered(self, parity: int, rows: int, cols: int):
        off = _FLAG_BYTES + parity * self.in_bytes
        n = rows * cols * self._local_bytes.new_empty((), dtype=self.dtype).element_size()
        return self._local_bytes[off : off + n].view(self.dtype).view(rows, cols)

    def _local_ptr(self, idx: int) -> ctypes.c_void_p:
        # local int arrays of 64 entries: [1] chunk arrival counters of the push role, [2] per-destination tile counters
        return ctypes.c_void_p(self.local.data_ptr() + idx * 4 * 64)

    # ------------------------------------------------------------------ ops
    def _next_epoch(self) -> int:
        """Advance the call counter on the host (for buffer parity) and on the device (the value kernels compare flags
        with).  The device increment is an ordinary stream operation, so a captured step replays correctly as long as
        the number of fused calls per replay is even (parity then repeats); see ``pad_to_even``."""
        self.epoch += 1
        self.epoch_dev.add_(1)
        return self.epoch

    def pad_to_even(self, calls_before: int):
        """Call at the end of a step that will be captured in a CUDA graph: if the step made an odd number of fused
        calls, spend one barrier so every replay starts on the same buffer parity."""
        if (self.epoch - calls_before) % 2:
            self.barrier()

    def barrier(self):
        """Device-side barrier over the group on the current stream (bounded wait)."""
        self._next_epoch()
        rc = _lib.cuda_lib().oslo_symm_barrier(
            self._flag_ptrs(2), ctypes.c_void_p(self.base + 2 * 256), ctypes.c_int(self.rank), ctypes.c_int(self.tp),
            ctypes.c_int(self.epoch), _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr(), _lib.ptr(self.epoch_dev))
        if rc:
            raise RuntimeError(f"oslo_symm_barrier failed ({rc})")

    def supports(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        if x.dtype != self.dtype or w.dtype != self.dtype or x.dim() != 2 or w.dim() != 2:
            return False
        rows, k = x.shape
        n = w.shape[0]
        if k % 8 or n % 8:
            return False
        # x is either a token shard (ag) or the full token set (rs); both must tile into 128-row blocks per rank
        return True

    def _weight_operand(self, w):
        if w.stride(-1) == 1:
            return w, 0, w.stride(0)
        if w.stride(0) == 1:
            return w, 1, w.stride(1)
        w = w.contiguous()
        return w, 0, w.stride(0)

    def ag_ok(self, x_shard, w) -> bool:
        tl, k = x_shard.shape
        return (self.supports(x_shard, w) and tl % 128 == 0 and tl * self.tp <= self.max_tokens
                and k <= self.max_features and tl * self.tp * k * x_shard.element_size() <= self.in_bytes)

    def rs_ok(self, x, w, along_n: bool = False) -> bool:
        t, _ = x.shape
        n = w.shape[0]
        if along_n:  # every rank keeps its rows, the columns are scattered
            return (self.supports(x, w) and t % 128 == 0 and n % self.tp == 0 and (n // self.tp) % 64 == 0
                    and t * n * x.element_size() <= self.slot_bytes)
        return (self.supports(x, w) and t % self.tp == 0 and (t // self.tp) % 128 == 0 and t <= self.max_tokens
                and n <= self.max_features and t * n * x.element_size() <= self.slot_bytes)

    def ag_gemm(self, x_shard: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, keep: bool = True,
                gelu_grad_of: Optional[torch.Tensor] = None):
        """Returns ``(all_gather(x_shard) @ weight^T (+ bias, added in the epilogue), all_gather(x_shard))``.

        The gathered activations live in the workspace's symmetric buffer of this call's parity, which the peers
        overwrite two fused calls later.  ``keep=True`` (default) returns a private copy, e.g. to save for a backward
        pass; ``keep=False`` returns the view for consumers that are enqueued right away."""
        tl, k = x_shard.shape
        t = tl * self.tp
        n = weight.shape[0]
        self._next_epoch()
        parity = self.epoch & 1
        if not x_shard.is_contiguous() or x_shard.data_ptr() % 16:
            x_shard = x_shard.contiguous()
        out = torch.empty(t, n, dtype=x_shard.dtype, device=x_shard.device)
        w, b_mn, ldb = self._weight_operand(weight)
        if bias is not None:
            if bias.shape != (n,):
                raise ValueError("ag_gemm: bias must be [N]")
            bias = bias.to(x_shard.dtype).contiguous()
        if gelu_grad_of is not None:
            # the product is multiplied by gelu'(pre-activation) in the epilogue: [T, N], contiguous, operand dtype
            if gelu_grad_of.shape != (t, n) or gelu_grad_of.dtype != x_shard.dtype or not gelu_grad_of.is_contiguous() or bias is not None:
                raise ValueError("ag_gemm: gelu_grad_of must be a contiguous [T, N] tensor of the operand dtype, without bias")
        external = 0
        if self.ce_transport:
            self._ce_push_shard(x_shard, parity, tl, k)
            external = 1
        rc = _lib.cuda_lib().oslo_ag_gemm(
            _lib.ptr(x_shard), self._gathered_ptrs(parity), _lib.ptr(w), _lib.ptr(out), _lib.ptr(bias), ctypes.c_int(t),
            ctypes.c_int(n), ctypes.c_int(k), ctypes.c_longlong(ldb), ctypes.c_int(b_mn),
            ctypes.c_int(1 if self.dtype == torch.bfloat16 else 0), ctypes.c_int(self.tp), ctypes.c_int(self.rank),
            ctypes.c_int(self.epoch), self._flag_ptrs(0), self._local_ptr(1), ctypes.c_int(self.copy_ctas),
            ctypes.c_int(_lib.num_sms()), _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr(), _lib.ptr(self.epoch_dev),
            self._mc_gathered(parity), ctypes.c_int(external), _lib.ptr(gelu_grad_of))
        if rc:
            raise RuntimeError(f"oslo_ag_gemm failed ({rc})")
        if external:
            self._ce_join()
        x_full = self._local_gathered(parity, t, k)
        return out, (x_full.clone() if keep else x_full)

    # ------------------------------------------------------------ copy-engine transport
    def _ce_fork(self):
        """Side streams start after everything enqueued so far on the current stream (inputs ready, epoch advanced)."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        return ev

    def _ce_join(self):
        """The current stream continues only after our outgoing transfers: their sources may be reused afterwards."""
        main = torch.cuda.current_stream()
        for r, s in enumerate(self._ce_streams):
            if r != self.rank:
                main.wait_stream(s)

    def _flag_view(self, r: int, which: int) -> torch.Tensor:
        """int32 view of rank ``r``'s flag array ``which`` (0 chunk flags, 1 reduce-scatter flags), 64 entries."""
        return self._peer_bytes[r][which * 256 : which * 256 + 256].view(torch.int32)

    def _ce_push_shard(self, x_shard: torch.Tensor, parity: int, tl: int, k: int):
        """All-gather transport by copy engine: our shard goes into block [rank] of every rank's gathered buffer, row chunk
        by row chunk, each chunk followed by its flag (a 4-byte copy of the device-resident epoch), one stream per
        destination.  The consuming kernel runs meanwhile on the current stream and takes chunks as flags come up."""
        esz = x_shard.element_size()
        chunk_rows = _lib.cuda_lib().oslo_ag_chunk_rows(ctypes.c_int(tl), ctypes.c_int(self.tp))
        if chunk_rows <= 0:
            raise RuntimeError("all-gather chunking failed")
        cps = tl // chunk_rows
        chunk_bytes = chunk_rows * k * esz
        src = x_shard.view(torch.uint8).view(-1)
        base = _FLAG_BYTES + parity * self.in_bytes + self.rank * tl * k * esz
        ev = self._ce_fork()
        for i in range(1, self.tp + 1):
            d = (self.rank + i) % self.tp
            dst = self._peer_bytes[d]
            if d == self.rank:
                # our own block of the gathered buffer (callers get the whole gathered tensor back): a local copy
                dst[base : base + cps * chunk_bytes].copy_(src)
                continue
            stream = self._ce_streams[d]
            stream.wait_event(ev)
            flags = self._flag_view(d, 0)
            with torch.cuda.stream(stream):
                for c in range(cps):
                    dst[base + c * chunk_bytes : base + (c + 1) * chunk_bytes].copy_(src[c * chunk_bytes : (c + 1) * chunk_bytes])
                    flags[self.rank * cps + c : self.rank * cps + c + 1].copy_(self.epoch_dev)

    def _gemm_rs_ce(self, x, weight, bias, addend, pair):
        """Reduce-scatter transport by copy engine.  The product is computed block of rows by block of rows in destination
        order (next rank first, our own block last); each finished block leaves for its owner's slot [rank] on that
        destination's stream while the next block is multiplied, followed by its flag; our own block is summed with the
        other ranks' blocks, which have arrived in our slot buffer meanwhile, by a small kernel that waits on the flags."""
        from oslo_b200.ops.gemm import gemm

        t, k = x.shape
        n = weight.shape[0]
        tl = t // self.tp
        esz = x.element_size()
        self._next_epoch()
        parity = self.epoch & 1
        blk_bytes = tl * n * esz
        if self._stage is None or self._stage.numel() < 2 * blk_bytes:
            self._stage = torch.empty(2 * blk_bytes, dtype=torch.uint8, device=self.device)
            self._stage_free = [None, None]
        main = torch.cuda.current_stream()
        slot_base = _FLAG_BYTES + 2 * self.in_bytes + parity * self.slot_bytes
        out = torch.empty(tl, n, dtype=x.dtype, device=x.device)
        own = None
        for i in range(1, self.tp + 1):
            d = (self.rank + i) % self.tp
            rows = slice(d * tl, (d + 1) * tl)
            if d == self.rank:
                own = torch.empty(tl, n, dtype=x.dtype, device=x.device)
                part = own
            else:
                b = i & 1
                if self._stage_free[b] is not None:
                    main.wait_event(self._stage_free[b])  # the transfer that last read this staging buffer is done
                part = self._stage[b * blk_bytes : (b + 1) * blk_bytes].view(x.dtype).view(tl, n)
            if addend is not None:
                part.copy_(addend[rows])
                gemm(x[rows], weight, out=part, accumulate=True)
            else:
                gemm(x[rows], weight, out=part)
            if pair is not None:
                gemm(pair[0][rows], pair[1], out=part, accumulate=True)
            if d == self.rank:
                continue
            ev = self._ce_fork()
            stream = self._ce_streams[d]
            stream.wait_event(ev)
            with torch.cuda.stream(stream):
                off = slot_base + self.rank * blk_bytes
                self._peer_bytes[d][off : off + blk_bytes].copy_(part.view(torch.uint8).view(-1))
                self._flag_view(d, 1)[self.rank : self.rank + 1].copy_(self.epoch_dev)
                done = torch.cuda.Event()
                done.record(stream)
                self._stage_free[i & 1] = done
        rc = _lib.cuda_lib().oslo_rs_fold(
            _lib.ptr(own), ctypes.c_void_p(self.base + slot_base), ctypes.c_void_p(self.base + 256), ctypes.c_int(self.rank),
            ctypes.c_int(self.tp), ctypes.c_longlong(tl), ctypes.c_int(n), _lib.ptr(out), _lib.ptr(bias),
            ctypes.c_int(1 if self.dtype == torch.bfloat16 else 0), ctypes.c_int(self.epoch), _lib.ptr(self.epoch_dev),
            _lib.ptr(_lib.status_word(self.device)), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_rs_fold failed ({rc})")
        self._ce_join()
        return out

    def gemm_rs(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                addend: Optional[torch.Tensor] = None, along_n: bool = False, pair=None):
        """Returns this rank's block of ``reduce_scatter(x @ weight^T + addend)``: its rows (``[T/tp, N]``), or with
        ``along_n`` its columns (``[T, N/tp]``, the 2-D / 2.5-D layouts).  ``addend`` is an optional local ``[T, N]``
        partial product that rides along in the same reduce-scatter."""
        t, k = x.shape
        n = weight.shape[0]
        tl = t if along_n else t // self.tp
        if not x.is_contiguous():
            x = x.contiguous()
        if self.ce_transport and not along_n and tl * n * x.element_size() % 16 == 0:
            return self._gemm_rs_ce(x, weight, bias, addend, pair)
        if pair is not None:  # the in-kernel transports take the second product as a ready [T, N] addend
            from oslo_b200.ops.gemm import matmul_nt

            extra = matmul_nt(pair[0], pair[1])
            addend = extra if addend is None else addend + extra
        self._next_epoch()
        parity = self.epoch & 1
        out = torch.empty(tl, n // self.tp if along_n else n, dtype=x.dtype, device=x.device)
        w, b_mn, ldb = self._weight_operand(weight)
        if addend is not None:
            if addend.shape != (t, n) or addend.dtype != x.dtype:
                raise ValueError("gemm_rs: addend must be [T, N] in the operand dtype")
            addend = addend.contiguous()
        rc = _lib.cuda_lib().oslo_gemm_rs(
            _lib.ptr(x), ctypes.c_longlong(x.stride(0)), _lib.ptr(w), ctypes.c_longlong(ldb), ctypes.c_int(b_mn),
            _lib.ptr(out), _lib.ptr(bias), ctypes.c_int(t), ctypes.c_int(n), ctypes.c_int(k),
            ctypes.c_int(1 if self.dtype == torch.bfloat16 else 0), ctypes.c_int(self.tp), ctypes.c_int(self.rank),
            ctypes.c_int(self.epoch), self._slot_ptrs(parity), self._flag_ptrs(1), self._local_ptr(2),
            ctypes.c_int(self.copy_ctas), ctypes.c_int(_lib.num_sms()), _lib.ptr(_lib.status_word(self.device)),
            _lib.stream_ptr(), _lib.ptr(self.debug_times), _lib.ptr(self.epoch_dev), _lib.ptr(addend),
            ctypes.c_int(1 if along_n else 0), self._mc_slots(parity))
        if rc:
            raise RuntimeError(f"oslo_gemm_rs failed ({rc})")
        return out

    def ag_gemm_rs(self, rs_ws: "SymmetricWorkspace", x_shard: torch.Tensor, weight: torch.Tensor):
        """``reduce_scatter_rows over rs_ws's group ( all_gather_rows over this group (x_shard) @ weight^T )`` in one
        launch; returns ``(out [T / tp, N], gathered x [T, K])``.  Both groups must have the same size (they cut the
        rows into the same blocks), e.g. the INPUT and OUTPUT groups of 3-D tensor parallelism."""
        tl, k = x_shard.shape
        t = tl * self.tp
        n = weight.shape[0]
        if rs_ws.tp != self.tp:
            raise ValueError("ag_gemm_rs: the gather and scatter groups must have the same size")
        self._next_epoch()
        rs_ws._next_epoch()
        ag_par, rs_par = self.epoch & 1, rs_ws.epoch & 1
        if not x_shard.is_contiguous() or x_shard.data_ptr() % 16:
            x_shard = x_shard.contiguous()
        out = torch.empty(tl, n, dtype=x_shard.dtype, device=x_shard.device)
        w, b_mn, ldb = self._weight_operand(weight)
        rc = _lib.cuda_lib().oslo_ag_gemm_rs(
            _lib.ptr(x_shard), self._gathered_ptrs(ag_par), _lib.ptr(w), ctypes.c_longlong(ldb), ctypes.c_int(b_mn), _lib.ptr(out),
            ctypes.c_int(t), ctypes.c_int(n), ctypes.c_int(k), ctypes.c_int(1 if self.dtype == torch.bfloat16 else 0),
            ctypes.c_int(self.tp), ctypes.c_int(self.rank), ctypes.c_int(self.epoch), self._flag_ptrs(0),
            self._local_ptr(1), _lib.ptr(self.epoch_dev),
            ctypes.c_int(rs_ws.tp), ctypes.c_int(rs_ws.rank), ctypes.c_int(rs_ws.epoch), rs_ws._slot_ptrs(rs_par),
            rs_ws._flag_ptrs(1), rs_ws._local_ptr(2), _lib.ptr(rs_ws.epoch_dev),
            ctypes.c_int(self.copy_ctas), ctypes.c_int(_lib.num_sms()), _lib.ptr(_lib.status_word(self.device)),
            _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_ag_gemm_rs failed ({rc})")
        return out, self._local_gathered(ag_par, t, k).clone()

    def ag_rs_ok(self, rs_ws, x_shard, w) -> bool:
        tl, k = x_shard.shape
        t, n = tl * self.tp, w.shape[0]
        return (self.ag_ok(x_shard, w) and rs_ws is not None and rs_ws.tp == self.tp
                and t * n * x_shard.element_size() <= rs_ws.slot_bytes)


class _Runtime:
    """Adapter registered with :mod:`oslo_b200.ops.fused_collectives`."""

    def __init__(self, ws: SymmetricWorkspace):
        self.ws = ws

    def supports(self, x, w):
        if x.dim() != 2:
            return False
        # called with either a token shard (all-gather side) or full tokens (reduce-scatter side)
        return self.ws.ag_ok(x, w) or self.ws.rs_ok(x, w)

    def ag_gemm(self, x_shard, weight, bias=None, keep=True, gelu_grad_of=None):
        if not self.ws.ag_ok(x_shard, weight):
            raise RuntimeError("ag_gemm: operands not supported by the fused kernel")
        return self.ws.ag_gemm(x_shard, weight, bias, keep, gelu_grad_of)

    def gemm_rs(self, x, weight, addend=None, along_n=False, pair=None):
        if not self.ws.rs_ok(x, weight, along_n):
            raise RuntimeError("gemm_rs: operands not supported by the fused kernel")
        return self.ws.gemm_rs(x, weight, addend=addend, along_n=along_n, pair=pair)


def enable(pc, mode, max_tokens: int, max_features: int, dtype=torch.bfloat16, copy_ctas: int = 16, model=None,
           multimem: bool = True, ce_transport: Optional[bool] = None) -> bool:
    """Create the group's symmetric workspace and switch the linears that communicate over ``mode`` to the fused kernels:
    ``TENSOR_1D`` for the sequence-parallel 1-D linears, ``TENSOR_2D_ROW`` / ``TENSOR_2P5D_ROW`` for the feature
    reduce-scatter of the SUMMA linears, ``TENSOR_3D_INPUT`` + ``TENSOR_3D_OUTPUT`` (call twice) for the 3-D linear.
    ``max_tokens x max_features`` bounds the product that one call may exchange.  With ``model`` given, its
    vocab-parallel embedding tables are moved to symmetric memory as well."""
    if not (torch.cuda.is_available() and pc.use_cuda) or pc.get_world_size(mode) == 1:
        return False
    if model is not None:
        rehome_vocab_embeddings(model, pc, mode)
    global _fused_small_ops
    ws = SymmetricWorkspace(pc, mode, max_tokens, max_features, dtype, copy_ctas, multimem=multimem, ce_transport=ce_transport)
    fused_collectives.set_runtime(_Runtime(ws), mode)
    _fused_small_ops = True
    return True


def disable():
    global _fused_small_ops
    fused_collectives.clear_runtimes()
    _fused_small_ops = False
