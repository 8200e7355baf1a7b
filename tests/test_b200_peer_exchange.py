"""The in-kernel exchange of sharded reductions, as far as ONE GPU can show it.

Two ranks' kernels that wait for each other must not share a GPU, so the multi-rank exchange itself is
tested on two GPUs (tests/test_shard_gloo.py, NCCL variant). Here a group of ONE rank runs the same
code path - the result goes through the window and back - and a group that claims a second rank which
never writes shows that the wait is bounded and reported, not a hang.
"""

import numpy as np
import pytest

from harness import lcg_data
from pytorches_b200 import abi
from pytorches_b200.core import Device, Tensor
from pytorches_b200.shard import ShardGroup

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 5, 1000, 70_001, 1 << 20, (1 << 22) + 3])
def test_single_rank_group_gives_the_plain_results(b200, n):
    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange(), b200.last_error()
    x = (np.round(lcg_data(n, 9) * 64) / 64).astype(np.float32)
    x[n // 3] = 7.0
    x[n - 1] = 7.0
    t = Tensor.from_numpy(x, dev)
    bits = lambda a: np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    for _ in range(6):  # more reductions than slot generations
        assert bits(g.sum(t).numpy()) == bits(t.sum().numpy())
        assert bits(g.mean(t, n).numpy()) == bits(t.mean().numpy())
        assert bits(g.max(t).numpy()) == bits(t.max().numpy())
        assert g.argmax(t, 1000).numpy() == n // 3 + 1000


@pytest.mark.parametrize("rows,cols", [(37, 24), (1000, 4096), (0, 64), (5, 1), (300, 1000)])
def test_single_rank_group_column_sums_through_the_window(b200, rows, cols):
    """A vector result (a bias gradient) goes through the window's vector area and back: the bits of SUM_AXIS(0)."""
    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange(), b200.last_error()
    x = lcg_data(rows * cols, 5).reshape(rows, cols)
    t = Tensor.from_numpy(x, dev)
    want = t.raw_sum_axis(0).numpy() if rows else np.zeros(cols, dtype=np.float32)
    for _ in range(6):  # more than there are slot generations
        got = g.sum_axis0(t).numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("n", [70_001, (1 << 22) + 3])
def test_pointers_inside_a_buffer_take_the_narrow_load_kernels(b200, n):
    """The extension entry points accept any 4-byte aligned f32 pointer, not only the start of a plugin
    buffer. A pointer that is not 16-byte aligned must not reach the bulk-copy or 128-bit-load kernels
    (a misaligned access would be a device fault, not a status): it takes the narrow-load forms, whose
    results carry the same bits. A pointer that is not even 4-byte aligned is refused."""
    import ctypes as C

    lib = b200.lib
    reduce_ = lib.pytorches_b200_peer_reduce
    reduce_.restype, reduce_.argtypes = C.c_int32, [C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_int64, C.c_uint64, C.c_void_p]
    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange(), b200.last_error()
    x = (np.round(lcg_data(n + 3, 11) * 64) / 64).astype(np.float32)
    whole = Tensor.from_numpy(x, dev)
    for shift in (1, 2, 3):  # elements: 4, 8, 12 bytes into the buffer
        view = Tensor.from_numpy(x[shift:shift + n], dev)  # the same values at an aligned address
        want = [view.sum().numpy(), view.max().numpy(), view.argmax().numpy()]
        for kind, w in zip((0, 1, 2), want):
            out = Tensor.zeros_on([2], dev)
            assert reduce_(0, kind, whole.buffer.ptr + 4 * shift, n, 0, 1000 + shift * 3 + kind, out.buffer.ptr) == abi.STATUS_OK, b200.last_error()
            got = out.numpy()
            if kind == 2:
                assert int(got.view(np.int64)[0]) == int(w)
            else:
                assert got.view(np.uint32)[0] == np.float32(w).reshape(1).view(np.uint32)[0], (kind, shift, got[0], w)
    out = Tensor.zeros_on([2], dev)
    assert reduce_(0, 0, whole.buffer.ptr + 2, n, 0, 2000, out.buffer.ptr) == abi.STATUS_INVALID_ARGUMENT
    b200.synchronize(0)


@pytest.mark.parametrize("n", [65536, 65536 * 3 + 5, 65536 * 200, (1 << 24) + 65536 * 3 + 1])
def test_single_rank_group_sums_in_unsplit_order(b200, n):
    """The sharded sum 'in unsplit order' with one rank: every block sum goes through the window's block
    area and the chain over them must give SUM_AXIS's bits, call after call (more calls than generations)."""
    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange(), b200.last_error()
    assert g.unsplit_order(n)
    t = Tensor.from_numpy(lcg_data(n, 13), dev)
    for _ in range(6):
        assert g.sum(t, 0, n).numpy().tobytes() == t.sum().numpy().tobytes()
        assert g.mean(t, n, 0).numpy().tobytes() == t.mean().numpy().tobytes()


def test_unsplit_order_with_more_blocks_than_one_copy_holds(b200):
    """4797 blocks (an odd number, a ragged last block): the combiner's bulk copies hold 4096 words, so
    the window over the block sums has to move; the bits must still be SUM_AXIS's."""
    n = 65536 * 4096 + 65536 * 700 + 3
    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange(), b200.last_error()
    assert g.unsplit_order(n)
    t = Tensor.rand_uniform_on([n], 21, -1.0, 1.0, dev)
    for _ in range(3):
        assert g.sum(t, 0, n).numpy().tobytes() == t.sum().numpy().tobytes()
        assert g.mean(t, n, 0).numpy().tobytes() == t.mean().numpy().tobytes()


def test_unsplit_order_needs_whole_blocks(b200):
    import ctypes as C

    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 2)  # two ranks on paper: only the rule is asked here
    g._peer_reduce = object()
    assert g.unsplit_order(65536 * 8) and g.unsplit_order(65536 * 8 + 2 * 17) is False  # 2 x (4 blocks + 17): rank 1 would start inside a block
    assert not g.unsplit_order(65536)  # rank 1 would hold nothing
    fn = b200.lib.pytorches_b200_peer_sum_unsplit
    fn.restype = C.c_int32
    fn.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_void_p]
    t = Tensor.from_numpy(lcg_data(70000, 1), dev)
    out = Tensor.zeros_on([1], dev)
    assert fn(0, t.buffer.ptr, 70000, 100, 1 << 20, 0, 0, out.buffer.ptr) == abi.STATUS_INVALID_ARGUMENT and "65536" in b200.last_error()


def test_column_sums_wider_than_the_window_are_refused(b200):
    import ctypes as C

    fn = b200.lib.pytorches_b200_peer_sum_axis0
    fn.restype, fn.argtypes = C.c_int32, [C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]
    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange()
    t = Tensor.from_numpy(lcg_data(2 * 4097, 1).reshape(2, 4097), dev)
    out = Tensor.zeros_on([4097], dev)
    assert fn(0, t.buffer.ptr, 2, 4097, 0, out.buffer.ptr) == abi.STATUS_INVALID_ARGUMENT and "4096" in b200.last_error()
    assert g.sum_axis0(t).numpy().shape == (4097,)  # the shard layer falls back to its gather-and-combine path


def test_a_peer_that_never_answers_is_a_reported_error_not_a_hang(b200):
    import ctypes as C

    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange()
    # Claim a second rank whose window is this same memory: nothing ever writes rank 1's slot.
    lib = b200.lib
    handle = C.create_string_buffer(64)
    assert lib.pytorches_b200_peer_export(0, handle) == 0
    assert lib.pytorches_b200_peer_attach(0, 0, 2, handle.raw + handle.raw, 50) == 0  # give up after 50 ms
    t = Tensor.from_numpy(lcg_data(1 << 20, 3), dev)
    out = g.sum(t)  # enqueued; the kernel waits 50 ms, records the failure and returns
    with pytest.raises(abi.PluginError) as err:
        b200.synchronize(0)
    assert err.value.status == abi.STATUS_INTERNAL and "peer" in str(err.value)
    b200.synchronize(0)  # reported once; the device is usable
    assert g.enable_peer_exchange()  # a fresh one-rank group works again
    assert g.sum(t).numpy() == t.sum().numpy()
    del out


def test_unsplit_sum_whose_peer_never_sends_its_blocks_is_a_reported_error(b200):
    """The same for a sum in unsplit order: the combiner's copies of the block sums keep coming back
    without the second rank's words; after the time limit the failure is recorded, not waited out."""
    import ctypes as C

    dev = Device(b200, 0)
    g = ShardGroup(dev, 0, 1)
    assert g.enable_peer_exchange()
    lib = b200.lib
    handle = C.create_string_buffer(64)
    assert lib.pytorches_b200_peer_export(0, handle) == 0
    assert lib.pytorches_b200_peer_attach(0, 0, 2, handle.raw + handle.raw, 50) == 0  # two ranks on paper, 50 ms of patience
    fn = lib.pytorches_b200_peer_sum_unsplit
    fn.restype = C.c_int32
    fn.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_void_p]
    n = 65536 * 40
    t = Tensor.from_numpy(lcg_data(n, 5), dev)
    out = Tensor.zeros_on([1], dev)
    assert fn(0, t.buffer.ptr, n, 0, 2 * n, 0, g.peer_seq, out.buffer.ptr) == abi.STATUS_OK, b200.last_error()  # blocks 40..79 never come
    g.advance_peer_seq(g.peer_seq + 1)
    with pytest.raises(abi.PluginError) as err:
        b200.synchronize(0)
    assert err.value.status == abi.STATUS_INTERNAL and "peer" in str(err.value)
    b200.synchronize(0)  # reported once; the device is usable
    assert g.enable_peer_exchange()
    assert g.sum(t, 0, n).numpy().tobytes() == t.sum().numpy().tobytes()


def test_peer_reduce_needs_attached_windows(b200):
    import ctypes as C

    lib = b200.lib
    fn = lib.pytorches_b200_peer_attach
    fn.restype, fn.argtypes = C.c_int32, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_char_p, C.c_uint32]
    assert fn(0, 3, 2, b"\0" * 128, 0) == abi.STATUS_INVALID_ARGUMENT  # rank outside the group
    assert fn(0, 0, 9, b"\0" * 64 * 9, 0) == abi.STATUS_INVALID_ARGUMENT  # more ranks than a window has slots
