"""Sharding mode for the hot path: one process per GPU, tensors split along their leading dimension.

The reference has no multi-device execution of one op; its planner only places whole layers on
devices (``crates/core/src/strategy.rs:221-326``) and moves tensors through host memory
(``crates/core/src/lib.rs:535-542``). This module is the sharding mode the hot path needs instead:

* elementwise ops run on each rank's rows with no communication (operands whose leading dimension is
  broadcast are simply replicated);
* a reduction that crosses the leading dimension runs locally to a per-rank partial, the partials are
  all-gathered (the only exchange: a few bytes per rank), and every rank combines them IN RANK ORDER
  with the same plugin op it used locally. The combine is therefore deterministic and identical on
  all ranks, like the reference's fixed-order block combine (``plugins/cpu/src/reduce.rs:1-4``).

``torch.distributed`` is the plumbing (NCCL over NVLink on GPUs, gloo on CPU); every arithmetic step,
including the combine, is a plugin op on the device's in-order stream.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .abi import DTYPE_F32, DTYPE_I64, KIND_CUDA, Arg, contiguous_strides, op
from .core import Buffer, Device, Operand, Tensor, run_op_into


def split_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """(first row, row count) of ``rank``'s shard: rows are dealt out evenly, earlier ranks take the remainder."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def split_layers(n_layers: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous blocks of whole layers per rank, the reference's layer-split placement applied to the
    optimizer update (crates/core/src/strategy.rs:269-326). Same dealing rule as ``split_rows``."""
    return split_rows(n_layers, rank, world)


def nccl_options():
    """Process-group options for the exchanges of this path: partials of 4 to 12 bytes per rank.

    Left alone, NCCL sizes its kernels for bandwidth: at 8 ranks an all-gather occupies many CTAs that
    spin on their peers while the next local pass is streaming on the same GPU, and that pass loses
    the SMs they hold. One CTA moves these few bytes just as fast. ``PYTORCHES_B200_NCCL_CTAS=0``
    keeps the library's own choice (for comparison); any other number is the CTA limit.

    The exchange is meant to run BESIDE the next local pass, but both become runnable at the same
    moment and the pass has thousands of CTAs queued: at equal priority the collective's one CTA can
    wait behind all of them, so it starts when the pass ends and its latency (which grows with the
    number of ranks) is paid in full. The communication stream is therefore a high-priority stream:
    its CTA takes the first slot that frees up. ``PYTORCHES_B200_NCCL_PRIORITY=0`` turns that off."""
    import os

    # The exchanges are a few bytes per rank: in-switch reduction gains nothing, and a rank that exits
    # early while its memory is bound to an NVLink multicast object can fault its peers' GPUs.
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    ctas = int(os.environ.get("PYTORCHES_B200_NCCL_CTAS", "1"))
    high = os.environ.get("PYTORCHES_B200_NCCL_PRIORITY", "1") != "0"
    opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=high)
    if ctas > 0:
        opts.config.min_ctas = 1
        opts.config.max_ctas = ctas
    return opts


class _CudaView:
    """Exposes a device allocation of the plugin through ``__cuda_array_interface__`` (no copy)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


class ShardGroup:
    """One rank's handle on a sharded computation."""

    def __init__(self, device: Device, rank: int = 0, world: int = 1, group: Optional[dist.ProcessGroup] = None):
        self.device, self.rank, self.world, self.group = device, rank, world, group
        self.is_cuda = device.plugin.device_info(device.index).kind == KIND_CUDA
        self._stream = None
        self._pending: list = []  # combines not yet enqueued: (collectives to wait for, what to enqueue)
        self._views: dict = {}  # (pointer, elements, dtype) -> torch alias; the allocator hands the same blocks out again
        self._peer_reduce = None  # set by enable_peer_exchange: full-tensor reductions then exchange inside their kernel
        self._peer_seq = 0
        if self.is_cuda and world > 1:
            fn = device.plugin.lib.pytorches_b200_stream
            fn.restype, fn.argtypes = C.c_void_p, [C.c_uint32]
            self._stream = torch.cuda.ExternalStream(fn(device.index), device=torch.device("cuda", device.index))
            # Collectives order themselves against torch's CURRENT stream. A rank process of a sharded
            # run has one job, so the plugin's stream is made current once, for good, instead of
            # entering a stream context around every collective (that costs more host time per step
            # than the collectives themselves).
            torch.cuda.set_stream(self._stream)

    # ---- in-kernel exchange over peer memory ----
    def enable_peer_exchange(self, wait_ms: int = 0) -> bool:
        """Switches the full-tensor reductions (``sum``, ``mean``, ``max``, ``argmax``) from "local pass,
        NCCL all-gather, combine op" to ONE launch per reduction: the kernel that finishes the local
        pass stores this GPU's result into every rank's peer-mapped window over NVLink, waits (bounded:
        ``wait_ms``, default 2 s) for the other ranks' results to land in its own window and combines
        them in rank order. Same bits as the NCCL path. Only the B200 plugin has this (its extension
        entry points ``pytorches_b200_peer_*``); ranks are processes on one node, at most 8. Collective:
        every rank must call it; returns False (and changes nothing) unless it worked on all of them."""
        lib = self.device.plugin.lib
        if not self.is_cuda or not hasattr(lib, "pytorches_b200_peer_reduce") or self.world > 8:
            ok = False
        else:
            export, attach, reduce_ = lib.pytorches_b200_peer_export, lib.pytorches_b200_peer_attach, lib.pytorches_b200_peer_reduce
            export.restype, export.argtypes = C.c_int32, [C.c_uint32, C.c_void_p]
            attach.restype, attach.argtypes = C.c_int32, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_char_p, C.c_uint32]
            reduce_.restype = C.c_int32
            reduce_.argtypes = [C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_int64, C.c_uint64, C.c_void_p]
            mean_ = lib.pytorches_b200_peer_mean
            mean_.restype, mean_.argtypes = C.c_int32, [C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]
            self._peer_mean = mean_
            uns_ = lib.pytorches_b200_peer_sum_unsplit
            uns_.restype = C.c_int32
            uns_.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_void_p]
            self._peer_sum_unsplit = uns_
            vec_ = lib.pytorches_b200_peer_sum_axis0
            vec_.restype, vec_.argtypes = C.c_int32, [C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]
            self._peer_sum_axis0 = vec_
            self.flush()
            handle = C.create_string_buffer(64)
            ok = export(self.device.index, handle) == 0
        mine = handle.raw if ok else b""
        if self.world > 1:
            every = [None] * self.world
            dist.all_gather_object(every, mine, group=self.group)
        else:
            every = [mine]
        ok = all(len(h) == 64 for h in every)
        if ok:
            ok = attach(self.device.index, self.rank, self.world, b"".join(every), wait_ms) == 0
        if self.world > 1:  # all or nothing: a rank that could not map its peers must not leave the others waiting for it
            flags = [None] * self.world
            dist.all_gather_object(flags, ok, group=self.group)
            ok = all(flags)
        self._peer_reduce, self._peer_seq = (reduce_ if ok else None), 0
        return ok

    def disable_peer_exchange(self) -> None:
        """Back to the NCCL exchange (every rank must do the same before its next reduction)."""
        self._peer_reduce = None

    @property
    def peer_exchange(self) -> bool:
        return self._peer_reduce is not None

    def _peer(self, kind: int, x_local: Tensor, first_index: int = 0, n_total: int = 0) -> Tensor:
        """kind 0 sum, 1 max, 2 argmax, 3 mean (``n_total`` = element count of the whole tensor)."""
        dev = self.device
        out = Tensor(Buffer(dev, 1, 8 if kind == 2 else 4), [], dtype=DTYPE_I64 if kind == 2 else DTYPE_F32)
        seq, self._peer_seq = self._peer_seq, self._peer_seq + 1  # ranks issue the same reductions in the same order
        if kind == 3:
            status = self._peer_mean(dev.index, x_local.buffer.ptr, x_local.numel(), n_total, seq, out.buffer.ptr)
        else:
            status = self._peer_reduce(dev.index, kind, x_local.buffer.ptr, x_local.numel(), first_index, seq, out.buffer.ptr)
        dev.plugin.check(status, "sharded reduction with in-kernel exchange")
        note = getattr(dev.plugin, "peer_reduce", None)  # a recorder writes the call down (replay.Recorder)
        if note is not None:
            note(dev.index, kind, x_local.buffer.ptr, x_local.numel(), first_index, n_total, out.buffer.ptr, out.dtype)
        return out

    def peer_trace(self) -> np.ndarray:
        """[64, 16] device-clock readings (ns) of this rank's last 64 reductions with an in-kernel exchange,
        row (seq % 0xfffffffe + 1) % 64: [1] own part complete, [2] every rank's part arrived, [3] result
        written; for sums in unsplit order also [13], how many bulk copies of the block sums the combiner
        needed (``pytorches_b200_peer_trace``; all zero unless PYTORCHES_B200_PEER_TRACE=1).
        Synchronizes the device's stream."""
        fn = self.device.plugin.lib.pytorches_b200_peer_trace
        fn.restype, fn.argtypes = C.c_int32, [C.c_uint32, C.c_void_p]
        out = np.zeros((64, 16), dtype=np.uint64)
        self.device.plugin.check(fn(self.device.index, out.ctypes.data), "peer trace")
        return out

    def advance_peer_seq(self, to: int) -> None:
        """After a replayed list issued sharded reductions natively: the next one continues from ``to``."""
        self._peer_seq = to

    @property
    def peer_seq(self) -> int:
        return self._peer_seq

    # ---- plumbing ----
    def torch_view(self, t: Tensor) -> torch.Tensor:
        """A torch tensor aliasing ``t``'s device memory, for handing to a collective."""
        n = t.numel()
        key = (t.buffer.ptr, n, t.dtype)
        view = self._views.get(key)
        if view is None:
            if len(self._views) > 256:
                self._views.clear()
            if self.is_cuda:
                typestr = "<i8" if t.dtype == DTYPE_I64 else "<f4"
                view = torch.as_tensor(_CudaView(t.buffer.ptr, (n,), typestr), device=torch.device("cuda", self.device.index))
            else:
                ctype = C.c_int64 if t.dtype == DTYPE_I64 else C.c_float
                view = torch.from_numpy(np.ctypeslib.as_array((ctype * n).from_address(t.buffer.ptr)))
            self._views[key] = view
        return view

    def _gather_async(self, t: Tensor):
        """Starts the all-gather of ``t`` behind everything enqueued so far; returns (gathered tensor, work or None)."""
        itemsize = 8 if t.dtype == DTYPE_I64 else 4
        out = Tensor(Buffer(self.device, self.world * t.numel(), itemsize), [self.world] + list(t.shape), dtype=t.dtype)
        if self.world == 1:
            self.device.plugin.copy_device_to_device(self.device.index, out.buffer.ptr, t.buffer.ptr, t.numel() * itemsize)
            return out, None
        src, dst = self.torch_view(t), self.torch_view(out)
        return out, dist.all_gather_into_tensor(dst, src, group=self.group, async_op=True)

    def _wait(self, work) -> None:
        """Orders the device's stream (on CPU: the host) behind a collective started by ``_gather_async``."""
        if work is not None:
            work.wait()  # on a GPU this is a stream-side wait: the host does not block

    def all_gather(self, t: Tensor) -> Tensor:
        """[world, *t.shape]: row r holds rank r's ``t``. The collective is enqueued on the device's stream."""
        out, work = self._gather_async(t)
        self._wait(work)
        return out

    # ---- deferred combines ----
    # A sharded reduction is: local pass, exchange of the partials, combine. The exchange is latency, not
    # bandwidth; to hide it, the combine of one reduction is enqueued only after the local pass of the
    # NEXT one, so the collective runs (on the communication library's stream) beside that pass. Results
    # are ``_Deferred`` tensors: touching their storage, or calling ``flush``, enqueues what is pending.
    def flush(self) -> None:
        pending, self._pending = self._pending, []
        for works, finish in pending:
            for w in works:
                self._wait(w)
            finish()

    def _defer(self, local_pass, shape, dtype, finish_into) -> Tensor:
        """``local_pass()`` -> list of partial tensors (enqueued now); ``finish_into(gathered, out_buffer)``
        enqueues the combine later. Returns the tensor the combine will write."""
        partials = local_pass()
        self.flush()  # earlier reductions' collectives have had this local pass to hide behind
        gathered, works = [], []
        for part in partials:
            g, w = self._gather_async(part)
            gathered.append(g)
            works.append(w)
        out_buf = Buffer(self.device, math.prod(shape), 8 if dtype == DTYPE_I64 else 4)
        keep = partials  # the collective reads them: keep them allocated until it has been waited for
        self._pending.append((works, lambda: (finish_into(gathered, out_buf), keep.clear())))
        return _Deferred(self, out_buf, shape, dtype)

    # ---- reductions that cross the sharded (leading) dimension ----
    def _combine(self, code: int, out_dtype=DTYPE_F32):
        def finish(gathered, out_buf):
            g = gathered[0]
            run_op_into(self.device, code, [0], [Operand.contiguous(g)], out_buf, g.shape[1:], out_dtype)
        return finish

    PEER_VECTOR_MAX = 4096  # elements of a result the in-kernel exchange carries (pytorches_b200_peer_sum_axis0)

    def sum_axis0(self, x_local: Tensor) -> Tensor:
        """Sum over the sharded leading dimension: local SUM_AXIS(0), all-gather, SUM_AXIS(0) in rank order.
        With the in-kernel exchange enabled and a result of at most 4096 elements (a bias gradient), the
        per-rank sums travel through the peer windows instead and no collective library is involved."""
        m = math.prod(x_local.shape[1:])
        if self._peer_reduce and 0 < m <= self.PEER_VECTOR_MAX:
            dev = self.device
            out = Tensor(Buffer(dev, m), list(x_local.shape[1:]))
            seq, self._peer_seq = self._peer_seq, self._peer_seq + 1
            dev.plugin.check(self._peer_sum_axis0(dev.index, x_local.buffer.ptr, x_local.shape[0] if x_local.shape else 1, m, seq, out.buffer.ptr),
                             "sharded column sum with in-kernel exchange")
            return out
        return self._defer(lambda: [x_local.raw_sum_axis(0)], x_local.shape[1:], DTYPE_F32, self._combine(op.SUM_AXIS))

    SUM_BLOCK = 65536        # the reference's summation block (plugins/cpu/src/reduce.rs:10)
    UNSPLIT_MAX_BLOCKS = 16384

    def unsplit_order(self, n_total: int) -> bool:
        """Whether a sum over a tensor of ``n_total`` elements, split by ``split_rows`` over this group,
        can be computed with the bits of the UNSPLIT sum: the in-kernel exchange is on, every shard is a
        run of whole 65536-element blocks and holds at least one. The same answer on every rank."""
        import os

        if os.environ.get("PYTORCHES_B200_UNSPLIT_ORDER", "1") == "0":  # diagnostic: keep the rank-ordered combine
            return False
        if not self._peer_reduce or n_total <= 0 or -(-n_total // self.SUM_BLOCK) > self.UNSPLIT_MAX_BLOCKS:
            return False
        for r in range(self.world):
            start, count = split_rows(n_total, r, self.world)
            if count == 0 or start % self.SUM_BLOCK or (start + count != n_total and count % self.SUM_BLOCK):
                return False
        return True

    def _peer_unsplit(self, x_local: Tensor, first_index: int, n_total: int, mean: bool) -> Tensor:
        dev = self.device
        out = Tensor(Buffer(dev, 1), [])
        seq, self._peer_seq = self._peer_seq, self._peer_seq + 1
        dev.plugin.check(self._peer_sum_unsplit(dev.index, x_local.buffer.ptr, x_local.numel(), first_index, n_total, 1 if mean else 0, seq,
                                                out.buffer.ptr), "sharded sum in unsplit order")
        note = getattr(dev.plugin, "peer_reduce", None)  # a recorder writes the call down (replay.Recorder)
        if note is not None:
            note(dev.index, 5 if mean else 4, x_local.buffer.ptr, x_local.numel(), first_index, n_total, out.buffer.ptr, out.dtype)
        return out

    def sum(self, x_local: Tensor, first_index: Optional[int] = None, n_total: Optional[int] = None) -> Tensor:
        """Full-tensor sum. Given where this rank's shard starts in the flattened tensor and the
        tensor's size, and shards of whole 65536-element blocks (``unsplit_order``), every rank chains
        ALL block sums in block order: the bits of the sum over the unsplit tensor, whatever the number
        of ranks. Otherwise every rank's ``Tensor.sum`` partial, combined in rank order."""
        if first_index is not None and n_total is not None and self.unsplit_order(n_total):
            return self._peer_unsplit(x_local, first_index, n_total, False)
        if self._peer_reduce:
            return self._peer(0, x_local)
        return self._defer(lambda: [x_local.raw_reshape([x_local.numel()]).raw_sum_axis(0)], [], DTYPE_F32, self._combine(op.SUM_AXIS))

    def mean(self, x_local: Tensor, n_global: int, first_index: Optional[int] = None) -> Tensor:
        """``Tensor.mean`` of the reference: the sum, then a DIV by the element count as a scalar tensor.
        With ``first_index`` and block-aligned shards the sum is taken in unsplit order (see ``sum``)."""
        if first_index is not None and self.unsplit_order(n_global):
            return self._peer_unsplit(x_local, first_index, n_global, True)
        if self._peer_reduce:  # the DIV by the f32 count runs in the combining kernel: the same bits, one launch instead of three
            return self._peer(3, x_local, 0, n_global)

        def finish(gathered, out_buf):
            total = gathered[0].raw_sum_axis(0)
            count = Tensor.scalar_on(float(n_global), self.device)
            run_op_into(self.device, op.DIV, [0], [Operand.contiguous(total), Operand.contiguous(count)], out_buf, [])
        return self._defer(lambda: [x_local.raw_reshape([x_local.numel()]).raw_sum_axis(0)], [], DTYPE_F32, finish)

    def max(self, x_local: Tensor) -> Tensor:
        if self._peer_reduce:
            return self._peer(1, x_local)
        return self._defer(lambda: [x_local.raw_reshape([x_local.numel()]).raw_reduce_axis(op.MAX_AXIS, 0)], [], DTYPE_F32,
                           self._combine(op.MAX_AXIS))

    def argmax(self, x_local: Tensor, first_index: int) -> Tensor:
        """Position of the maximum in the unsharded flattened tensor; ``first_index`` is where this
        rank's shard starts in it. One pass yields (max, position); the pairs are gathered and the best
        is picked on every rank (NCCL has no pair reduction)."""
        if self._peer_reduce:
            return self._peer(2, x_local, first_index)
        dev = self.device

        def local_pass():
            flat = x_local.raw_reshape([x_local.numel()])
            val = Tensor(Buffer(dev, 1), [])
            idx = Tensor(Buffer(dev, 1, 8), [], dtype=DTYPE_I64)
            dev.plugin.execute(dev.index, op.MAX_ARGMAX_AXIS, [0, first_index],
                               [Arg(flat.buffer.ptr, tuple(flat.shape), tuple(contiguous_strides(flat.shape)))],
                               [Arg(val.buffer.ptr, (), ()), Arg(idx.buffer.ptr, (), (), DTYPE_I64)])
            return [val, idx]

        def finish(gathered, out_buf):
            run_op_into(dev, op.ARGMAX_COMBINE, [0], [Operand.contiguous(gathered[0]), Operand.contiguous(gathered[1])], out_buf, [], DTYPE_I64)

        return self._defer(local_pass, [], DTYPE_I64, finish)


class _Deferred(Tensor):
    """Result of a sharded reduction whose combine may not have been enqueued yet. Reading its storage
    (any op or read-back does) first enqueues everything its group has pending."""

    def __init__(self, group: ShardGroup, buffer: Buffer, shape, dtype):
        self._group, self._buf = group, buffer
        super().__init__(buffer, shape, dtype=dtype)

    @property
    def buffer(self) -> Buffer:
        self._group.flush()
        return self._buf

    @buffer.setter
    def buffer(self, value: Buffer) -> None:
        self._buf = value
