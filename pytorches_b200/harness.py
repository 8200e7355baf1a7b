"""Shared helpers of the conformance checks and the tests: drive any plugin at the vtable, the way plugins/cpu/tests/kernels.rs does.

``lcg_data`` is that file's ``data()`` generator (kernels.rs:13-21), ``exec_op`` its ``exec`` helper
(kernels.rs:59-66), ``close`` its tolerance rule (kernels.rs:68-74).
"""

from __future__ import annotations

import numpy as np

from pytorches_b200.abi import DTYPE_F32, DTYPE_I64, Arg, Plugin, contiguous_strides

MASK64 = (1 << 64) - 1


def lcg_data(n: int, seed: int) -> np.ndarray:
    """Deterministic f32 values in [-1, 1): the stream of kernels.rs:13-21, computed in O(log n) numpy
    passes by prefix doubling of the LCG's affine map (checked against a scalar loop in the tests)."""
    a, c = 6364136223846793005, 1442695040888963407
    s0 = np.uint64((seed * a + c) & MASK64)
    with np.errstate(over="ignore"):
        mult = np.empty(n, dtype=np.uint64)
        add = np.empty(n, dtype=np.uint64)
        if n:
            mult[0], add[0] = np.uint64(a), np.uint64(c)
        filled = 1
        while filled < n:
            take = min(filled, n - filled)
            # map for index filled+i = map[filled-1] composed after map[i]
            m_hi, d_hi = mult[filled - 1], add[filled - 1]
            mult[filled:filled + take] = mult[:take] * m_hi
            add[filled:filled + take] = add[:take] * m_hi + d_hi
            filled += take
        out = mult * s0 + add
    return ((out >> np.uint64(40)).astype(np.float32) / np.float32(8388608.0)) - np.float32(1.0)


class Buf:
    """A device buffer filled from host data (kernels.rs:23-47)."""

    def __init__(self, plugin: Plugin, host: np.ndarray, device: int = 0):
        self.plugin, self.device = plugin, device
        self.host_dtype = host.dtype
        host = np.ascontiguousarray(host)
        self.n = host.size
        self.nbytes = max(host.nbytes, 4)
        self.ptr = plugin.alloc(device, self.nbytes)
        if host.nbytes:
            plugin.copy_from_host(device, self.ptr, host.ctypes.data, host.nbytes)

    @staticmethod
    def empty(plugin: Plugin, n: int, dtype=np.float32, device: int = 0) -> "Buf":
        fill = np.full(n, np.nan, dtype=np.float32) if dtype == np.float32 else np.full(n, -7, dtype=dtype)
        return Buf(plugin, fill, device)

    def get(self) -> np.ndarray:
        out = np.empty(self.n, dtype=self.host_dtype)
        if out.nbytes:
            self.plugin.copy_to_host(self.device, out.ctypes.data, self.ptr, out.nbytes)
        return out

    def free(self):
        if self.ptr is not None:
            self.plugin.free(self.device, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def exec_op(plugin: Plugin, code: int, ints, ins, out: Buf, oshape, out_dtype=DTYPE_F32, device: int = 0) -> int:
    """``ins`` = [(Buf, shape, strides)]. Returns the status (kernels.rs:59-66)."""
    args = [Arg(b.ptr, tuple(sh), tuple(st)) for (b, sh, st) in ins]
    o = Arg(out.ptr, tuple(oshape), tuple(contiguous_strides(oshape)), out_dtype)
    return plugin.execute_status(device, code, list(ints), args, [o])


def close(what: str, got: np.ndarray, want: np.ndarray, rtol: float) -> None:
    """abs err <= rtol * max|want|, or both NaN, or equal (kernels.rs:68-74)."""
    assert got.shape == want.shape, f"{what}: length {got.shape} vs {want.shape}"
    if want.size == 0:
        return
    scale = max(float(np.nanmax(np.abs(want))) if np.isfinite(want).any() else 0.0, 1e-30)
    with np.errstate(invalid="ignore"):
        ok = (np.abs(got - want) <= np.float32(rtol * scale)) | (np.isnan(got) & np.isnan(want)) | (got == want)
    bad = np.flatnonzero(~ok)
    assert bad.size == 0, f"{what}[{bad[0]}]: got {got.reshape(-1)[bad[0]]}, want {want.reshape(-1)[bad[0]]} ({bad.size} bad)"


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_equal(what: str, got: np.ndarray, want: np.ndarray, zero_sign_matters: bool = True) -> None:
    """Bit-for-bit equality; NaNs compare equal to NaNs whatever their payload."""
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    g, w = bits(got), bits(want)
    same = g == w
    same |= np.isnan(got) & np.isnan(want)
    if not zero_sign_matters:
        same |= (got == 0) & (want == 0)
    bad = np.flatnonzero(~same.reshape(-1))
    assert bad.size == 0, (
        f"{what}: {bad.size} of {g.size} differ; first at {bad[0]}: got {got.reshape(-1)[bad[0]]!r} "
        f"(0x{g.reshape(-1)[bad[0]]:08x}), want {want.reshape(-1)[bad[0]]!r} (0x{w.reshape(-1)[bad[0]]:08x})")


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two f32 arrays (NaN vs NaN = 0, else huge)."""
    ia = bits(a).astype(np.int64)
    ib = bits(b).astype(np.int64)
    ia = np.where(ia & 0x80000000, 0x80000000 - ia, ia)  # map to a monotonic integer line
    ib = np.where(ib & 0x80000000, 0x80000000 - ib, ib)
    d = np.abs(ia - ib)
    both_nan = np.isnan(a) & np.isnan(b)
    one_nan = np.isnan(a) ^ np.isnan(b)
    d = np.where(both_nan, 0, d)
    return np.where(one_nan, 1 << 40, d)


def strided_view_numpy(storage: np.ndarray, shape, strides) -> np.ndarray:
    """The logical tensor an (shape, element strides) operand denotes over flat ``storage``."""
    return np.lib.stride_tricks.as_strided(storage, shape=tuple(shape), strides=tuple(s * storage.itemsize for s in strides))
