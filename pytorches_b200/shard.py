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
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .abi import DTYPE_F32, DTYPE_I64, KIND_CUDA, Arg, contiguous_strides, op
from .core import Buffer, Device, Operand, Tensor, run_op


def split_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """(first row, row count) of ``rank``'s shard: rows are dealt out evenly, earlier ranks take the remainder."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def split_layers(n_layers: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous blocks of whole layers per rank, the reference's layer-split placement applied to the
    optimizer update (crates/core/src/strategy.rs:269-326). Same dealing rule as ``split_rows``."""
    return split_rows(n_layers, rank, world)


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
        if self.is_cuda and world > 1:
            fn = device.plugin.lib.pytorches_b200_stream
            fn.restype, fn.argtypes = C.c_void_p, [C.c_uint32]
            self._stream = torch.cuda.ExternalStream(fn(device.index), device=torch.device("cuda", device.index))

    # ---- plumbing ----
    def torch_view(self, t: Tensor) -> torch.Tensor:
        """A torch tensor aliasing ``t``'s device memory, for handing to a collective."""
        n = t.numel()
        if self.is_cuda:
            typestr = "<i8" if t.dtype == DTYPE_I64 else "<f4"
            return torch.as_tensor(_CudaView(t.buffer.ptr, (n,), typestr), device=torch.device("cuda", self.device.index))
        ctype = C.c_int64 if t.dtype == DTYPE_I64 else C.c_float
        return torch.from_numpy(np.ctypeslib.as_array((ctype * n).from_address(t.buffer.ptr)))

    def all_gather(self, t: Tensor) -> Tensor:
        """[world, *t.shape]: row r holds rank r's ``t``. The collective is enqueued on the device's stream."""
        out = Tensor(Buffer(self.device, self.world * t.numel(), 8 if t.dtype == DTYPE_I64 else 4), [self.world] + list(t.shape), dtype=t.dtype)
        if self.world == 1:
            self.device.plugin.copy_device_to_device(self.device.index, out.buffer.ptr, t.buffer.ptr, t.numel() * (8 if t.dtype == DTYPE_I64 else 4))
            return out
        src, dst = self.torch_view(t), self.torch_view(out)
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                dist.all_gather_into_tensor(dst, src, group=self.group)
        else:
            dist.all_gather_into_tensor(dst, src, group=self.group)
        return out

    # ---- reductions that cross the sharded (leading) dimension ----
    def sum_axis0(self, x_local: Tensor) -> Tensor:
        """Sum over the sharded leading dimension: local SUM_AXIS(0), all-gather, SUM_AXIS(0) in rank order."""
        return self.all_gather(x_local.raw_sum_axis(0)).raw_sum_axis(0)

    def sum(self, x_local: Tensor) -> Tensor:
        """Full-tensor sum: every rank's ``Tensor.sum`` partial, combined in rank order."""
        partial = x_local.raw_reshape([x_local.numel()]).raw_sum_axis(0)
        return self.all_gather(partial).raw_sum_axis(0)

    def mean(self, x_local: Tensor, n_global: int) -> Tensor:
        """``Tensor.mean`` of the reference: the sum, then a DIV by the element count as a scalar tensor."""
        return self.sum(x_local).raw_binary(Tensor.scalar_on(float(n_global), self.device), op.DIV)

    def max(self, x_local: Tensor) -> Tensor:
        partial = x_local.raw_reshape([x_local.numel()]).raw_reduce_axis(op.MAX_AXIS, 0)
        return self.all_gather(partial).raw_reduce_axis(op.MAX_AXIS, 0)

    def argmax(self, x_local: Tensor, first_index: int) -> Tensor:
        """Position of the maximum in the unsharded flattened tensor; ``first_index`` is where this
        rank's shard starts in it. One pass yields (max, position); the pairs are gathered and the best
        is picked on every rank (NCCL has no pair reduction)."""
        flat = x_local.raw_reshape([x_local.numel()])
        val = Tensor(Buffer(self.device, 1), [])
        idx = Tensor(Buffer(self.device, 1, 8), [], dtype=DTYPE_I64)
        dev = self.device
        dev.plugin.execute(dev.index, op.MAX_ARGMAX_AXIS, [0, first_index],
                           [Arg(flat.buffer.ptr, tuple(flat.shape), tuple(contiguous_strides(flat.shape)))],
                           [Arg(val.buffer.ptr, (), ()), Arg(idx.buffer.ptr, (), (), DTYPE_I64)])
        vals, idxs = self.all_gather(val), self.all_gather(idx)
        return run_op(dev, op.ARGMAX_COMBINE, [0], [Operand.contiguous(vals), Operand.contiguous(idxs)], [], DTYPE_I64)
