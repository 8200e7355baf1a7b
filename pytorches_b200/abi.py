"""ctypes binding of the pytorches plugin ABI (major version 4).

This is the reference-side binding a host would write: it mirrors, field for field, the structs and
the vtable of ``crates/plugin-abi/src/lib.rs`` (restated in C in ``include/pytorches_plugin_abi.h``)
and applies the loader's checks of ``crates/core/src/plugin.rs:76-90`` (``check_vtable``). It binds
ANY conforming plugin by path; nothing here knows which plugin it talks to.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from dataclasses import dataclass

ABI_VERSION = 4
ENTRY_SYMBOL = "pytorches_plugin_entry"

STATUS_OK, STATUS_UNSUPPORTED, STATUS_OUT_OF_MEMORY, STATUS_INVALID_ARGUMENT, STATUS_INTERNAL = range(5)
STATUS_NAMES = {0: "OK", 1: "UNSUPPORTED", 2: "OUT_OF_MEMORY", 3: "INVALID_ARGUMENT", 4: "INTERNAL"}

DTYPE_F32 = 0
DTYPE_I64 = 1  # appended: output of ARGMAX_AXIS only

KIND_CPU, KIND_CUDA = 0, 1
MEMORY_UNKNOWN = 2**64 - 1


class op:
    """Op codes (crates/plugin-abi/src/lib.rs:67-115); 203-206 and 501-503 are appended codes."""

    NEG, EXP, LOG, RELU, TANH, STEP = 1, 2, 3, 4, 5, 6
    ADD, SUB, MUL, DIV = 100, 101, 102, 103
    MATMUL, SUM_AXIS, MATMUL_T = 200, 201, 202
    MAX_AXIS, ARGMAX_AXIS = 203, 204
    MAX_ARGMAX_AXIS, ARGMAX_COMBINE = 205, 206  # appended, for sharded reductions
    COPY = 300
    FILL, RAND_NORMAL = 400, 401
    RAND_UNIFORM = 402  # appended: lo + scale * u from the RAND_NORMAL counter hash
    AXPY = 500
    RELU_GRAD, ADD_RELU, SUB_EXP = 501, 502, 503  # appended: optional fused ops, each equal to its two-op sequence


class TensorDesc(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("dtype", C.c_uint32),
        ("ndim", C.c_uint32),
        ("shape", C.POINTER(C.c_uint64)),
        ("strides", C.POINTER(C.c_uint64)),
    ]


class OpAttrs(C.Structure):
    _fields_ = [("ints", C.c_int64 * 4)]


class DeviceInfo(C.Structure):
    _fields_ = [
        ("name", C.c_char * 64),
        ("kind", C.c_uint32),
        ("total_memory", C.c_uint64),
        ("free_memory", C.c_uint64),
        ("flags", C.c_uint32),
    ]


_COPY = C.CFUNCTYPE(C.c_int32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_size_t)


class PluginVTable(C.Structure):
    _fields_ = [
        ("abi_version", C.c_uint32),
        ("struct_size", C.c_uint32),
        ("plugin_version", C.c_uint32),
        ("name", C.c_char_p),
        ("device_count", C.CFUNCTYPE(C.c_uint32)),
        ("device_info", C.CFUNCTYPE(C.c_int32, C.c_uint32, C.POINTER(DeviceInfo))),
        ("alloc", C.CFUNCTYPE(C.c_int32, C.c_uint32, C.c_size_t, C.POINTER(C.c_void_p))),
        ("free", C.CFUNCTYPE(None, C.c_uint32, C.c_void_p)),
        ("copy_from_host", _COPY),
        ("copy_to_host", _COPY),
        ("copy_device_to_device", _COPY),
        ("supports_op", C.CFUNCTYPE(C.c_uint32, C.c_uint32)),
        (
            "execute",
            C.CFUNCTYPE(
                C.c_int32, C.c_uint32, C.c_uint32, C.POINTER(OpAttrs),
                C.POINTER(TensorDesc), C.c_uint32, C.POINTER(TensorDesc), C.c_uint32,
            ),
        ),
        ("synchronize", C.CFUNCTYPE(C.c_int32, C.c_uint32)),
        ("last_error", C.CFUNCTYPE(C.c_char_p)),
    ]


assert C.sizeof(TensorDesc) == 32 and C.sizeof(OpAttrs) == 32 and C.sizeof(DeviceInfo) == 96
assert C.sizeof(PluginVTable) == 112


class PluginError(RuntimeError):
    """A plugin call returned a non-OK status. ``status`` holds the code.

    The reference core maps OUT_OF_MEMORY to a memory error and UNSUPPORTED / INVALID_ARGUMENT to an
    invalid-argument error (crates/core/src/lib.rs:101-111); subclasses below keep that split.
    """

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class PluginOutOfMemory(PluginError, MemoryError):
    pass


class PluginInvalid(PluginError, ValueError):
    pass


def contiguous_strides(shape) -> list[int]:
    st, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        st[i] = acc
        acc *= shape[i]
    return st


@dataclass
class Arg:
    """One operand of ``execute``: a device handle read through a shape and element strides."""

    data: int
    shape: tuple
    strides: tuple
    dtype: int = DTYPE_F32


class Plugin:
    """A loaded plugin: the vtable plus thin, checked wrappers around each entry point."""

    def __init__(self, path: str):
        path = os.path.abspath(path)
        if not os.path.exists(path):
            raise FileNotFoundError(f"plugin library not found: {path}")
        self.path = path
        self.lib = C.CDLL(path, mode=C.RTLD_LOCAL)
        entry = getattr(self.lib, ENTRY_SYMBOL)
        entry.restype = C.POINTER(PluginVTable)
        entry.argtypes = []
        ptr = entry()
        if not ptr:
            raise RuntimeError(f"{path}: {ENTRY_SYMBOL} returned NULL")
        self.vt = ptr.contents
        # check_vtable, crates/core/src/plugin.rs:76-90
        if self.vt.abi_version != ABI_VERSION:
            raise RuntimeError(f"{path}: ABI {self.vt.abi_version}, host needs {ABI_VERSION}")
        if self.vt.struct_size < C.sizeof(PluginVTable):
            raise RuntimeError(f"{path}: vtable of {self.vt.struct_size} bytes is too small")
        self.name = self.vt.name.decode()
        # Reading a function pointer out of the ctypes struct builds a new callable every time: do it once.
        self._alloc, self._free, self._execute = self.vt.alloc, self.vt.free, self.vt.execute
        self._supports_op, self._supports = self.vt.supports_op, {}
        self._tls = threading.local()  # per-thread descriptor cache: entry points may be called from any thread

    # ---- devices ----
    def device_count(self) -> int:
        return int(self.vt.device_count())

    def device_info(self, device: int = 0) -> DeviceInfo:
        info = DeviceInfo()
        self.check(self.vt.device_info(device, C.byref(info)), "device_info")
        return info

    def last_error(self) -> str:
        msg = self.vt.last_error()
        return msg.decode(errors="replace") if msg else ""

    def check(self, status: int, what: str) -> None:
        if status == STATUS_OK:
            return
        msg = f"{what}: {self.last_error()}"
        if status == STATUS_OUT_OF_MEMORY:
            raise PluginOutOfMemory(status, msg)
        if status in (STATUS_UNSUPPORTED, STATUS_INVALID_ARGUMENT):
            raise PluginInvalid(status, msg)
        raise PluginError(status, msg)

    # ---- memory ----
    def alloc(self, device: int, nbytes: int) -> int:
        out = C.c_void_p()
        self.check(self._alloc(device, nbytes, C.byref(out)), f"alloc of {nbytes} bytes")
        return out.value or 0

    def free(self, device: int, handle: int) -> None:
        self._free(device, handle)

    def copy_from_host(self, device: int, dst: int, src_addr: int, nbytes: int) -> None:
        self.check(self.vt.copy_from_host(device, dst, src_addr, nbytes), "copy_from_host")

    def copy_to_host(self, device: int, dst_addr: int, src: int, nbytes: int) -> None:
        self.check(self.vt.copy_to_host(device, dst_addr, src, nbytes), "copy_to_host")

    def copy_device_to_device(self, device: int, dst: int, src: int, nbytes: int) -> None:
        self.check(self.vt.copy_device_to_device(device, dst, src, nbytes), "copy_device_to_device")

    def synchronize(self, device: int = 0) -> None:
        self.check(self.vt.synchronize(device), "synchronize")

    def supports_op(self, code: int) -> bool:
        known = self._supports.get(code)
        if known is None:
            known = self._supports[code] = bool(self._supports_op(code))  # a plugin's answer never changes
        return known

    # ---- execute ----
    _dims_cache: dict = {}

    @classmethod
    def _dims(cls, values: tuple):
        """A ctypes u64 array for a shape or stride tuple (cached: the same few tuples recur on a hot path)."""
        arr = cls._dims_cache.get(values)
        if arr is None:
            if len(cls._dims_cache) > 4096:
                cls._dims_cache.clear()
            arr = cls._dims_cache[values] = (C.c_uint64 * max(len(values), 1))(*values)
        return arr

    @classmethod
    def _desc(cls, a: Arg, keep: list) -> TensorDesc:
        return TensorDesc(a.data, a.dtype, len(a.shape), cls._dims(tuple(a.shape)), cls._dims(tuple(a.strides)))

    def execute_status(self, device: int, code: int, ints, inputs: list[Arg], outputs: list[Arg]) -> int:
        """Raw ``execute``: returns the status without raising (used by error-path tests)."""
        # The descriptor arrays for one call signature (shapes, strides, dtypes) are built once and
        # reused; only the data pointers and the attribute block change from call to call. Host time
        # per op matters: the ops of this path run for tens of microseconds on the device.
        key = (tuple((tuple(a.shape), tuple(a.strides), a.dtype) for a in inputs),
               tuple((tuple(a.shape), tuple(a.strides), a.dtype) for a in outputs))
        cache = self._tls.__dict__.setdefault("calls", {})
        slot = cache.get(key)
        if slot is None:
            if len(cache) > 4096:
                cache.clear()
            keep: list = []
            ins = (TensorDesc * max(len(inputs), 1))(*[self._desc(a, keep) for a in inputs])
            outs = (TensorDesc * max(len(outputs), 1))(*[self._desc(a, keep) for a in outputs])
            attrs = OpAttrs()
            slot = cache[key] = (ins, outs, attrs, C.byref(attrs))
        ins, outs, attrs, attrs_ref = slot
        for i, a in enumerate(inputs):
            ins[i].data = a.data
        for i, a in enumerate(outputs):
            outs[i].data = a.data
        for i in range(4):
            attrs.ints[i] = ints[i] if i < len(ints) else 0
        return int(self._execute(device, code, attrs_ref, ins, len(inputs), outs, len(outputs)))

    def execute(self, device: int, code: int, ints, inputs: list[Arg], outputs: list[Arg]) -> None:
        self.check(self.execute_status(device, code, ints, inputs, outputs), f"op {code}")
