"""Recording a step's plugin calls once and replaying them from native code.

The reference core is native code: an op costs it a few microseconds of host time
(``crates/core/src/lib.rs:331-370``, ``benchmarks/README.md:98-99``). The Python mirror of it in
``core.py`` needs ten times that per op, which is more than many ops of this path run for on a B200.
To measure (and to run) a step at the speed a native host would drive it, ``Recorder`` wraps a
plugin, lets one real step run through it, and writes down every ``alloc``, ``free``, ``execute`` and
sharded reduction of that step, call for call, with result buffers named by slot instead of by
address. ``RecordedStep.run(k)`` hands the list to the plugin's ``pytorches_b200_replay`` entry point
(``include/pytorches_b200_ext.h``), which issues it k times through the same entry points the vtable
exposes. Nothing is fused, reordered or skipped: the device sees the calls the host made.
"""

from __future__ import annotations

import ctypes as C
import math

from .abi import Plugin

CALL_EXECUTE, CALL_ALLOC, CALL_FREE, CALL_PEER_REDUCE = range(4)


class Operand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("slot", C.c_int32), ("dtype", C.c_uint32), ("ndim", C.c_uint32), ("reserved", C.c_uint32),
                ("shape", C.c_uint64 * 8), ("strides", C.c_uint64 * 8)]


class Call(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("op", C.c_uint32), ("ints", C.c_int64 * 4), ("n_in", C.c_uint32), ("n_out", C.c_uint32),
                ("ins", Operand * 2), ("outs", Operand * 2)]


assert C.sizeof(Operand) == 152 and C.sizeof(Call) == 656


class RecordedStep:
    """A call list ready to replay on ``device`` of ``plugin`` (the B200 plugin: it alone has the entry point)."""

    def __init__(self, plugin: Plugin, device: int, calls: list[Call], keep: list):
        self.plugin, self.device = plugin, device
        self.calls = (Call * max(len(calls), 1))(*calls)
        self.n = len(calls)
        self.keep = keep  # tensors whose memory the list names by address
        self.executes = sum(1 for c in calls if c.kind in (CALL_EXECUTE, CALL_PEER_REDUCE))
        self.peer_calls = sum(1 for c in calls if c.kind == CALL_PEER_REDUCE)
        self._fn = None

    def run(self, repeats: int = 1, first_seq: int = 0) -> int:
        """Issues the list ``repeats`` times; returns the sequence number after the last sharded reduction."""
        if self._fn is None:
            if not hasattr(self.plugin.lib, "pytorches_b200_replay"):
                raise RuntimeError(f"plugin '{self.plugin.name}' has no pytorches_b200_replay entry point")
            fn = self.plugin.lib.pytorches_b200_replay
            fn.restype, fn.argtypes = C.c_int32, [C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64]
            self._fn = fn
        self.plugin.check(self._fn(self.device, self.calls, self.n, repeats, first_seq), "replay")
        return first_seq + repeats * self.peer_calls


class Recorder:
    """Forwards to ``plugin`` and, between ``start`` and ``finish``, writes down what it forwards."""

    def __init__(self, plugin: Plugin):
        self._p = plugin
        self._recording = False
        self._calls: list[Call] = []
        self._slot_of: dict[int, int] = {}
        self._n_slots = 0

    def __getattr__(self, name):
        return getattr(self._p, name)

    # ---- control ----
    def start(self) -> None:
        self._recording, self._calls, self._slot_of, self._n_slots = True, [], {}, 0

    def finish(self, device: int, keep=()) -> RecordedStep:
        self._recording = False
        return RecordedStep(self._p, device, self._calls, list(keep))

    # ---- recorded entry points ----
    def alloc(self, device: int, nbytes: int) -> int:
        ptr = self._p.alloc(device, nbytes)
        if self._recording:
            slot, self._n_slots = self._n_slots, self._n_slots + 1
            self._slot_of[ptr] = slot
            c = Call(kind=CALL_ALLOC)
            c.ints[0], c.ints[1] = nbytes, slot
            self._calls.append(c)
        return ptr

    def free(self, device: int, handle: int) -> None:
        self._p.free(device, handle)
        if self._recording and handle in self._slot_of:
            c = Call(kind=CALL_FREE)
            c.ints[1] = self._slot_of.pop(handle)
            self._calls.append(c)

    def _operand(self, ptr: int, shape, strides, dtype: int) -> Operand:
        o = Operand(dtype=dtype, ndim=len(shape))
        slot = self._slot_of.get(ptr)
        o.slot = -1 if slot is None else slot
        o.data = None if slot is not None else ptr
        for i, (d, st) in enumerate(zip(shape, strides)):
            o.shape[i], o.strides[i] = d, st
        return o

    def execute(self, device: int, code: int, ints, inputs, outputs) -> None:
        if self._recording:
            if len(inputs) > 2 or len(outputs) > 2 or any(len(a.shape) > 8 for a in list(inputs) + list(outputs)):
                raise ValueError("a recorded call holds at most 2 inputs, 2 outputs and 8 dims")
            c = Call(kind=CALL_EXECUTE, op=code, n_in=len(inputs), n_out=len(outputs))
            for i in range(4):
                c.ints[i] = ints[i] if i < len(ints) else 0
            for i, a in enumerate(inputs):
                c.ins[i] = self._operand(a.data, a.shape, a.strides, a.dtype)
            for i, a in enumerate(outputs):
                c.outs[i] = self._operand(a.data, a.shape, a.strides, a.dtype)
            self._calls.append(c)
        self._p.execute(device, code, ints, inputs, outputs)

    def peer_reduce(self, device: int, kind: int, x_ptr: int, n: int, first_index: int, n_total: int, out_ptr: int, out_dtype: int) -> None:
        """Writes down a sharded reduction (``ShardGroup`` issues the real call itself)."""
        if self._recording:
            c = Call(kind=CALL_PEER_REDUCE, op=kind, n_in=1, n_out=1)
            c.ints[0], c.ints[1] = first_index, n_total
            c.ins[0] = self._operand(x_ptr, (n,), (1,), 0)
            c.outs[0] = self._operand(out_ptr, (), (), out_dtype)
            self._calls.append(c)


def algorithmic_bytes(step: RecordedStep) -> int:
    """Algorithmic bytes of one pass over the list: every distinct stored input of a call once, its
    outputs once (the reference's accounting, benchmarks/bench.py:166-170)."""
    total = 0
    for i in range(step.n):
        c = step.calls[i]
        if c.kind not in (CALL_EXECUTE, CALL_PEER_REDUCE):
            continue
        seen = set()
        for k in range(c.n_in):
            a = c.ins[k]
            key = (a.slot, a.data)
            if key in seen:
                continue
            seen.add(key)
            stored = math.prod(a.shape[d] for d in range(a.ndim) if a.strides[d] != 0) if a.ndim else 1
            total += stored * (8 if a.dtype == 1 else 4)
        for k in range(c.n_out):
            a = c.outs[k]
            total += (math.prod(a.shape[d] for d in range(a.ndim)) if a.ndim else 1) * (8 if a.dtype == 1 else 4)
    return total
