"""Host-side mirror of the reference core's tensor interface, for the hot path only.

The reference core (``crates/core/src/lib.rs``) turns tensor expressions into sequences of plugin
``execute`` calls: broadcasting becomes per-operand strides, every result is a fresh contiguous
buffer, and the backward pass is again plain ops (ReLU mask = STEP then MUL, broadcast gradient =
repeated SUM_AXIS, SGD = AXPY). This module replays exactly those sequences against any plugin that
exports the ABI, so a test written against it reads like the reference's own tests and exercises a
plugin the way the real core would. Method names and argument meaning follow the reference; each
cites the function it mirrors. It holds no kernels and no numeric code of its own.

Not in the reference (appended ops 203/204): ``sum_dim``, ``max_dim``, ``argmax_dim``, ``max``,
``argmax``. Also not in the reference: the optional fused ops 501-503 (``add_relu``, ``sub_exp`` and
the one-op relu gradient). They are used only on a device created with ``fused=True`` whose plugin
offers them (``supports_op``, as for ``axpy_``); otherwise, and by default, the two-op sequence of the
reference core runs. Either way the results carry the same bits.
"""

from __future__ import annotations

import ctypes as C
import math
import struct
from typing import Callable, Optional, Sequence

import numpy as np

from .abi import DTYPE_F32, DTYPE_I64, Arg, Plugin, contiguous_strides, op


def _f32_bits(v: float) -> int:
    return struct.unpack("<I", struct.pack("<f", v))[0]


class Device:
    """One device of one plugin (crates/core/src/lib.rs:141-186)."""

    def __init__(self, plugin: Plugin, index: int = 0, fused: bool = False):
        if index >= plugin.device_count():
            raise ValueError(f"{plugin.name}:{index} does not exist ({plugin.device_count()} devices)")
        self.plugin, self.index, self.fused = plugin, index, fused

    def __eq__(self, other):
        return isinstance(other, Device) and other.plugin is self.plugin and other.index == self.index

    def __hash__(self):
        return hash((id(self.plugin), self.index))

    def __str__(self):
        return f"{self.plugin.name}:{self.index}"

    def synchronize(self) -> None:
        self.plugin.synchronize(self.index)

    def supports_op(self, code: int) -> bool:
        return self.plugin.supports_op(code)

    def offers_fused(self, code: int) -> bool:
        """Whether an optional fused op (501-503) is to be used instead of its two-op sequence."""
        return self.fused and self.plugin.supports_op(code)


class Buffer:
    """Device storage owned through the plugin (crates/core/src/lib.rs:223-239)."""

    def __init__(self, device: Device, numel: int, itemsize: int = 4):
        self.device = device
        self.nbytes = max(numel * itemsize, 4)  # the core never asks for fewer than 4 bytes
        self.ptr = device.plugin.alloc(device.index, self.nbytes)

    def __del__(self):
        try:
            if self.ptr is not None:
                self.device.plugin.free(self.device.index, self.ptr)
                self.ptr = None
        except Exception:
            pass


class Node:
    def __init__(self, inputs: list["Tensor"], backward: Callable[["Tensor"], list[Optional["Tensor"]]]):
        self.inputs, self.backward = inputs, backward


def broadcast_shapes(a: Sequence[int], b: Sequence[int]) -> Optional[list[int]]:
    """NumPy-style broadcast (crates/core/src/lib.rs:286-301)."""
    n = max(len(a), len(b))
    pa, pb = n - len(a), n - len(b)
    out = []
    for i in range(n):
        da = 1 if i < pa else a[i - pa]
        db = 1 if i < pb else b[i - pb]
        if da == db or da == 1:
            out.append(db if da == 1 else da)
        elif db == 1:
            out.append(da)
        else:
            return None
    return out


def broadcast_strides(shape: Sequence[int], out_shape: Sequence[int]) -> list[int]:
    """Strides reading contiguous ``shape`` as ``out_shape``: 0 on broadcast dims (lib.rs:304-312)."""
    pad = len(out_shape) - len(shape)
    base = contiguous_strides(shape)
    st = [0] * len(out_shape)
    for i, d in enumerate(shape):
        st[pad + i] = 0 if d == 1 else base[i]
    return st


class Operand:
    """An op argument: a tensor read through an explicit shape/strides (lib.rs:315-329)."""

    def __init__(self, t: "Tensor", shape, strides):
        self.t, self.shape, self.strides = t, list(shape), list(strides)

    @staticmethod
    def contiguous(t: "Tensor") -> "Operand":
        return Operand(t, t.shape, contiguous_strides(t.shape))

    @staticmethod
    def broadcast(t: "Tensor", out_shape) -> "Operand":
        return Operand(t, out_shape, broadcast_strides(t.shape, out_shape))


def run_op_into(device: Device, code: int, ints, ins: list[Operand], out_buf: Buffer, out_shape, out_dtype=DTYPE_F32) -> None:
    """One ``execute`` into an existing contiguous buffer (crates/core/src/lib.rs:338-370)."""
    if not device.supports_op(code):
        raise ValueError(f"plugin '{device.plugin.name}' does not implement op {code}")
    for o in ins:
        if o.t.device != device:
            raise ValueError(f"tensors on different devices: {o.t.device} and {device}")
    args = [Arg(o.t.buffer.ptr, tuple(o.shape), tuple(o.strides), o.t.dtype) for o in ins]
    out = Arg(out_buf.ptr, tuple(out_shape), tuple(contiguous_strides(out_shape)), out_dtype)
    device.plugin.execute(device.index, code, list(ints), args, [out])


def run_op(device: Device, code: int, ints, ins: list[Operand], out_shape, out_dtype=DTYPE_F32) -> "Tensor":
    """Allocate the output, then ``run_op_into`` (crates/core/src/lib.rs:331-335)."""
    numel = math.prod(out_shape)
    buf = Buffer(device, numel, 8 if out_dtype == DTYPE_I64 else 4)
    run_op_into(device, code, ints, ins, buf, out_shape, out_dtype)
    return Tensor(buf, out_shape, dtype=out_dtype)


class Tensor:
    """A contiguous tensor on a plugin device with reverse-mode autograd (lib.rs:188-260)."""

    def __init__(self, buffer: Buffer, shape, requires_grad: bool = False, grad_fn: Optional[Node] = None, dtype: int = DTYPE_F32):
        self.buffer, self.shape = buffer, list(shape)
        self.requires_grad, self.grad_fn, self.dtype = requires_grad, grad_fn, dtype
        self.grad: Optional[Tensor] = None

    # ---- construction (lib.rs:379-470) ----
    @staticmethod
    def from_numpy(a: np.ndarray, device: Device, requires_grad: bool = False) -> "Tensor":
        a = np.ascontiguousarray(a, dtype=np.float32)
        buf = Buffer(device, a.size)
        if a.size:
            device.plugin.copy_from_host(device.index, buf.ptr, a.ctypes.data, a.nbytes)
        return Tensor(buf, a.shape, requires_grad)

    @staticmethod
    def full_on(shape, value: float, device: Device) -> "Tensor":
        return run_op(device, op.FILL, [_f32_bits(value)], [], list(shape))

    @staticmethod
    def ones_on(shape, device: Device) -> "Tensor":
        return Tensor.full_on(shape, 1.0, device)

    @staticmethod
    def zeros_on(shape, device: Device) -> "Tensor":
        return Tensor.full_on(shape, 0.0, device)

    @staticmethod
    def scalar_on(value: float, device: Device) -> "Tensor":
        return Tensor.full_on([], value, device)

    @staticmethod
    def randn_on(shape, seed: int, device: Device) -> "Tensor":
        return run_op(device, op.RAND_NORMAL, [seed], [], list(shape))

    @staticmethod
    def rand_uniform_on(shape, seed: int, lo: float, hi: float, device: Device, first: int = 0) -> "Tensor":
        """Uniform [lo, hi) from the counter hash (appended op RAND_UNIFORM, not in the reference):
        element i is lo + (hi - lo) * u(first + i)."""
        return run_op(device, op.RAND_UNIFORM, [seed, _f32_bits(lo), _f32_bits(hi - lo), first], [], list(shape))

    # ---- access ----
    @property
    def device(self) -> Device:
        return self.buffer.device

    def numel(self) -> int:
        return math.prod(self.shape)

    def numpy(self) -> np.ndarray:
        """Blocking read-back (``to_vec``, lib.rs:507-515)."""
        out = np.empty(self.shape, dtype=np.int64 if self.dtype == DTYPE_I64 else np.float32)
        if out.size:
            self.device.plugin.copy_to_host(self.device.index, out.ctypes.data, self.buffer.ptr, out.nbytes)
        return out

    def item(self):
        return self.numpy().reshape(-1)[0].item()

    def detach(self) -> "Tensor":
        return Tensor(self.buffer, self.shape, dtype=self.dtype)

    def requires_grad_(self, flag: bool = True) -> "Tensor":
        self.requires_grad = flag
        return self

    def attach(self, inputs: list["Tensor"], backward) -> "Tensor":
        if any(t.requires_grad for t in inputs):
            self.requires_grad = True
            self.grad_fn = Node(inputs, backward)
        return self

    # ---- raw (graph-free) kernels (lib.rs:546-591) ----
    def raw_unary(self, code: int) -> "Tensor":
        return run_op(self.device, code, [0], [Operand.contiguous(self)], self.shape)

    def raw_binary(self, o: "Tensor", code: int) -> "Tensor":
        out_shape = broadcast_shapes(self.shape, o.shape)
        if out_shape is None:
            raise ValueError(f"shapes {self.shape} and {o.shape} are not broadcastable")
        return run_op(self.device, code, [0], [Operand.broadcast(self, out_shape), Operand.broadcast(o, out_shape)], out_shape)

    def raw_reduce_axis(self, code: int, axis: int) -> "Tensor":
        shape = list(self.shape)
        del shape[axis]
        return run_op(self.device, code, [axis], [Operand.contiguous(self)], shape,
                      DTYPE_I64 if code == op.ARGMAX_AXIS else DTYPE_F32)

    def raw_sum_axis(self, axis: int) -> "Tensor":
        return self.raw_reduce_axis(op.SUM_AXIS, axis)

    def raw_reshape(self, shape) -> "Tensor":
        if math.prod(shape) != self.numel():
            raise ValueError(f"cannot reshape {self.shape} to {list(shape)}")
        return Tensor(self.buffer, shape, dtype=self.dtype)

    def raw_t(self) -> "Tensor":
        if len(self.shape) != 2:
            raise ValueError("t() needs a 2-D tensor")
        r, c = self.shape
        return run_op(self.device, op.COPY, [0], [Operand(self, [c, r], [1, c])], [c, r])

    def unbroadcast(self, target) -> "Tensor":
        """Reduce a broadcast result back to ``target`` by repeated SUM_AXIS (lib.rs:578-591)."""
        g = self
        while len(g.shape) > len(target):
            g = g.raw_sum_axis(0)
        for axis, dim in enumerate(target):
            if dim == 1 and g.shape[axis] != 1:
                keep = list(g.shape)
                keep[axis] = 1
                g = g.raw_sum_axis(axis).raw_reshape(keep)
        return g

    # ---- differentiable ops (lib.rs:595-670) ----
    def add(self, o: "Tensor") -> "Tensor":
        sa, sb = list(self.shape), list(o.shape)
        return self.raw_binary(o, op.ADD).attach([self, o], lambda g: [g.unbroadcast(sa), g.unbroadcast(sb)])

    def sub(self, o: "Tensor") -> "Tensor":
        sa, sb = list(self.shape), list(o.shape)
        return self.raw_binary(o, op.SUB).attach([self, o], lambda g: [g.unbroadcast(sa), g.neg().unbroadcast(sb)])

    def mul(self, o: "Tensor") -> "Tensor":
        a, b = self.detach(), o.detach()
        return self.raw_binary(o, op.MUL).attach(
            [self, o], lambda g: [g.mul(b).unbroadcast(a.shape), g.mul(a).unbroadcast(b.shape)])

    def div(self, o: "Tensor") -> "Tensor":
        a, b = self.detach(), o.detach()

        def back(g):
            gb = g.mul(a).div(b.mul(b)).neg()
            return [g.div(b).unbroadcast(a.shape), gb.unbroadcast(b.shape)]

        return self.raw_binary(o, op.DIV).attach([self, o], back)

    def neg(self) -> "Tensor":
        return self.raw_unary(op.NEG).attach([self], lambda g: [g.neg()])

    def exp(self) -> "Tensor":
        out = self.raw_unary(op.EXP)
        o = out.detach()
        return out.attach([self], lambda g: [g.mul(o)])

    def log(self) -> "Tensor":
        x = self.detach()
        return self.raw_unary(op.LOG).attach([self], lambda g: [g.div(x)])

    def relu(self) -> "Tensor":
        x = self.detach()
        return self.raw_unary(op.RELU).attach([self], lambda g: [g.relu_grad(x)])

    def relu_grad(self, x: "Tensor") -> "Tensor":
        """``self * step(x)``, the gradient of relu (lib.rs:639-643): RELU_GRAD when offered, else STEP then MUL."""
        if self.device.offers_fused(op.RELU_GRAD):
            return self.raw_binary(x, op.RELU_GRAD)
        return self.mul(x.raw_unary(op.STEP))

    # ---- fused forward ops (appended, optional): same values and gradients as the two ops they replace ----
    def add_relu(self, o: "Tensor") -> "Tensor":
        """``(self + o).relu()``: bias plus activation in one pass when the plugin offers ADD_RELU."""
        if not self.device.offers_fused(op.ADD_RELU):
            return self.add(o).relu()
        sa, sb = list(self.shape), list(o.shape)
        out = self.raw_binary(o, op.ADD_RELU)
        y = out.detach()  # step(relu(t)) == step(t): the output stands in for the pre-activation

        def back(g):
            gt = g.relu_grad(y)
            return [gt.unbroadcast(sa), gt.unbroadcast(sb)]

        return out.attach([self, o], back)

    def sub_exp(self, o: "Tensor") -> "Tensor":
        """``(self - o).exp()``, the numerator of a softmax, in one pass when the plugin offers SUB_EXP."""
        if not self.device.offers_fused(op.SUB_EXP):
            return self.sub(o).exp()
        sa, sb = list(self.shape), list(o.shape)
        out = self.raw_binary(o, op.SUB_EXP)
        y = out.detach()

        def back(g):
            gt = g.mul(y)
            return [gt.unbroadcast(sa), gt.neg().unbroadcast(sb)]

        return out.attach([self, o], back)

    def tanh(self) -> "Tensor":
        out = self.raw_unary(op.TANH)
        o = out.detach()
        return out.attach([self], lambda g: [g.mul(Tensor.scalar_on(1.0, g.device).sub(o.mul(o)))])

    def sum(self) -> "Tensor":
        shape = list(self.shape)
        out = self.raw_reshape([self.numel()]).raw_sum_axis(0)
        return out.attach([self], lambda g: [g.mul(Tensor.ones_on(shape, g.device))])

    def mean(self) -> "Tensor":
        shape, n = list(self.shape), float(self.numel())
        out = self.raw_reshape([self.numel()]).raw_sum_axis(0).raw_binary(Tensor.scalar_on(n, self.device), op.DIV)
        return out.attach(
            [self], lambda g: [g.mul(Tensor.ones_on(shape, g.device)).div(Tensor.scalar_on(n, g.device))])

    def t(self) -> "Tensor":
        return self.raw_t().attach([self], lambda g: [g.t()])

    def reshape(self, shape) -> "Tensor":
        old = list(self.shape)
        return self.raw_reshape(shape).attach([self], lambda g: [g.reshape(old)])

    def axpy_(self, alpha: float, other: "Tensor") -> None:
        """In-place ``self += alpha * other`` (lib.rs:709-720): AXPY when offered, else MUL+ADD+COPY."""
        if list(self.shape) != list(other.shape):
            raise ValueError(f"axpy_ shape mismatch: {self.shape} vs {other.shape}")
        dev = self.device
        if dev.supports_op(op.AXPY):
            run_op_into(dev, op.AXPY, [_f32_bits(alpha)], [Operand.contiguous(self), Operand.contiguous(other)], self.buffer, self.shape)
        else:
            scaled = other.raw_binary(Tensor.scalar_on(alpha, dev), op.MUL)
            upd = self.raw_binary(scaled, op.ADD)
            dev.plugin.copy_device_to_device(dev.index, self.buffer.ptr, upd.buffer.ptr, self.numel() * 4)

    # ---- appended reductions: no counterpart in the reference ----
    def sum_dim(self, axis: int, keepdim: bool = False) -> "Tensor":
        out = self.raw_sum_axis(axis)
        return out.raw_reshape(self._keep(axis)) if keepdim else out

    def max_dim(self, axis: int, keepdim: bool = False) -> "Tensor":
        out = self.raw_reduce_axis(op.MAX_AXIS, axis)
        return out.raw_reshape(self._keep(axis)) if keepdim else out

    def argmax_dim(self, axis: int, keepdim: bool = False) -> "Tensor":
        out = self.raw_reduce_axis(op.ARGMAX_AXIS, axis)
        return out.raw_reshape(self._keep(axis)) if keepdim else out

    def max(self) -> "Tensor":
        return self.raw_reshape([self.numel()]).raw_reduce_axis(op.MAX_AXIS, 0)

    def argmax(self) -> "Tensor":
        return self.raw_reshape([self.numel()]).raw_reduce_axis(op.ARGMAX_AXIS, 0)

    def _keep(self, axis: int) -> list[int]:
        keep = list(self.shape)
        keep[axis] = 1
        return keep

    # ---- operators ----
    def _coerce(self, o) -> "Tensor":
        return o if isinstance(o, Tensor) else Tensor.scalar_on(float(o), self.device)

    def __add__(self, o): return self.add(self._coerce(o))
    def __radd__(self, o): return self._coerce(o).add(self)
    def __sub__(self, o): return self.sub(self._coerce(o))
    def __rsub__(self, o): return self._coerce(o).sub(self)
    def __mul__(self, o): return self.mul(self._coerce(o))
    def __rmul__(self, o): return self._coerce(o).mul(self)
    def __truediv__(self, o): return self.div(self._coerce(o))
    def __rtruediv__(self, o): return self._coerce(o).div(self)
    def __neg__(self): return self.neg()

    # ---- autograd (lib.rs:735-788) ----
    def backward(self) -> None:
        if self.numel() != 1:
            raise ValueError("backward() needs a scalar tensor")
        if not self.requires_grad:
            raise ValueError("tensor does not require grad")
        order, visited, stack = [], set(), [(self, False)]
        while stack:  # iterative post-order DFS: inputs before consumers
            t, expanded = stack.pop()
            if expanded:
                order.append(t)
                continue
            if id(t) in visited:
                continue
            visited.add(id(t))
            stack.append((t, True))
            if t.grad_fn:
                for inp in t.grad_fn.inputs:
                    if inp.requires_grad and id(inp) not in visited:
                        stack.append((inp, False))
        grads = {id(self): Tensor.ones_on(self.shape, self.device)}
        for t in reversed(order):
            g = grads.pop(id(t), None)
            if g is None:
                continue
            if t.grad_fn:
                for inp, gi in zip(t.grad_fn.inputs, t.grad_fn.backward(g)):
                    if inp.requires_grad and gi is not None:
                        prev = grads.pop(id(inp), None)
                        grads[id(inp)] = prev.raw_binary(gi, op.ADD) if prev is not None else gi
            else:
                t.grad = t.grad.raw_binary(g, op.ADD) if t.grad is not None else g


class SGD:
    """``optim.SGD`` of the reference (crates/python/python/pytorches/optim.py:13-16): one AXPY per parameter."""

    def __init__(self, params: list[Tensor], lr: float):
        self.params, self.lr = list(params), lr

    def step(self) -> None:
        for p in self.params:
            if p.grad is not None:
                p.axpy_(-self.lr, p.grad)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None


def mse_loss(pred: Tensor, target: Tensor) -> Tensor:
    """``nn.mse_loss`` (crates/python/python/pytorches/nn.py:276-278): mean of the squared difference."""
    d = pred - target
    return (d * d).mean()
