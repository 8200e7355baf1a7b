"""The sharding layer on CPU: world_size 2 and 3 over gloo, with the CPU oracle as each rank's plugin.

Checks the host logic of ``pytorches_b200.shard``: row partitioning (uneven splits included),
elementwise ops on shards equal to the unsharded op, and reductions that cross the sharded dimension
equal to the fixed-order combine of the per-rank partials (bit-exact) and to the unsharded result
(exact for max/argmax, within the summation-order tolerance for sum/mean).
"""

import math
import os
import socket
import sys

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "pytorches_plugin_cpuref.so")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n: int, backend: str = "gloo"):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["PYTORCHES_CPU_THREADS"] = "2"
    from harness import lcg_data
    from pytorches_b200.abi import Plugin, op
    from pytorches_b200.core import Device, Tensor
    from pytorches_b200.shard import ShardGroup, nccl_options, split_rows

    if backend == "nccl":
        import torch

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=torch.device("cuda", rank), pg_options=nccl_options())
    else:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        # Expected values always come from the CPU oracle; the sharded computation runs on the plugin
        # under test (the oracle itself over gloo, the B200 plugin over NCCL: both must give the same bits).
        plugin = Plugin(ORACLE_SO)
        dev = Device(plugin, 0)
        if backend == "nccl":
            import pytorches_b200

            gdev = Device(pytorches_b200.load_plugin(), rank)
        else:
            gdev = dev
        g = ShardGroup(gdev, rank, world)
        bits = lambda a: np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)

        # ---- full-tensor reductions over n elements, ties and a clear maximum in a late shard ----
        x = (np.round(lcg_data(n, 7) * 32) / 32).astype(np.float32)
        x[n - 3] = 5.0
        x[n // 2] = 5.0  # the same maximum earlier: argmax must be the lower position, n // 2
        start, count = split_rows(n, rank, world)
        assert sum(split_rows(n, r, world)[1] for r in range(world)) == n
        local = Tensor.from_numpy(x[start:start + count], gdev)
        full = Tensor.from_numpy(x, dev)

        partials = []
        for r in range(world):  # every rank recomputes all partials locally to know the expected combine
            s, c = split_rows(n, r, world)
            partials.append(Tensor.from_numpy(x[s:s + c], dev).sum().numpy().reshape(1))
        want_sum = Tensor.from_numpy(np.concatenate(partials), dev).raw_sum_axis(0).numpy()
        got_sum = g.sum(local).numpy()
        assert bits(got_sum) == bits(want_sum), (got_sum, want_sum)
        ref = x.astype(np.float64).sum()
        assert abs(float(got_sum) - ref) <= 1e-5 * math.log2(n) * np.abs(x.astype(np.float64)).sum()
        got_mean = g.mean(local, n).numpy()
        assert bits(got_mean) == bits(np.float32(want_sum) / np.float32(n))

        assert bits(g.max(local).numpy()) == bits(full.max().numpy())
        assert g.argmax(local, start).numpy() == full.argmax().numpy() == n // 2

        # all ranks hold the same combined results
        gathered = [None] * world
        dist.all_gather_object(gathered, (got_sum.tobytes(), got_mean.tobytes()))
        assert all(item == gathered[0] for item in gathered)

        # ---- the same reductions with the exchange inside the kernels, over peer memory (B200 plugin only) ----
        if backend == "nccl":
            assert g.enable_peer_exchange(), gdev.plugin.last_error()
            for _ in range(3):  # several in a row: slot generations, epochs
                assert bits(g.sum(local).numpy()) == bits(want_sum)
                assert bits(g.mean(local, n).numpy()) == bits(np.float32(want_sum) / np.float32(n))
                assert bits(g.max(local).numpy()) == bits(full.max().numpy())
                assert g.argmax(local, start).numpy() == n // 2
            # Shards of whole 65536-element blocks: the sum is taken in UNSPLIT order and has the bits of the
            # oracle's sum over the whole tensor (and the mean those of its mean), several in a row.
            nb = 65536 * 2 * world * 3 + 777 if n > 1 << 20 else 0
            if nb:
                xb = lcg_data(nb, 19)
                per = 65536 * 2 * 3
                lo, cnt = (rank * per, per) if rank < world - 1 else (rank * per, nb - rank * per)
                class _Even(ShardGroup):  # the benchmark's even split: the last rank takes the ragged tail
                    def unsplit_order(self, n_total):
                        return self.peer_exchange
                ge = _Even.__new__(_Even)
                ge.__dict__.update(g.__dict__)
                shard = Tensor.from_numpy(xb[lo:lo + cnt], gdev)
                whole = Tensor.from_numpy(xb, dev)
                for _ in range(5):
                    assert bits(ge.sum(shard, lo, nb).numpy()) == bits(whole.sum().numpy())
                    assert bits(ge.mean(shard, nb, lo).numpy()) == bits(whole.mean().numpy())
                    assert ge.argmax(shard, lo).numpy() == whole.argmax().numpy()
                g._peer_seq = ge._peer_seq  # one sequence for the group: the next reduction continues it
            small = Tensor.from_numpy(x[start:start + 5], gdev)  # a shard too short for a combiner CTA: separate exchange launch
            want_small = sum((x[split_rows(n, r, world)[0]:][:5].astype(np.float64).sum() for r in range(world)))
            assert abs(float(g.sum(small).numpy()) - want_small) < 1e-4
            g.disable_peer_exchange()  # back to NCCL for what follows

        # ---- a [rows, cols] problem: elementwise on shards, then a column sum across shards ----
        rows, cols = 37, 24
        A = lcg_data(rows * cols, 1).reshape(rows, cols)
        b = lcg_data(cols, 2).reshape(1, cols)       # leading dim 1: replicated
        s_col = lcg_data(rows, 3).reshape(rows, 1)   # leading dim sharded like A
        r0, rc = split_rows(rows, rank, world)
        out_local = (Tensor.from_numpy(A[r0:r0 + rc], gdev) + Tensor.from_numpy(b, gdev)).relu() * Tensor.from_numpy(s_col[r0:r0 + rc], gdev)
        out_full = (Tensor.from_numpy(A, dev) + Tensor.from_numpy(b, dev)).relu() * Tensor.from_numpy(s_col, dev)
        assert np.array_equal(bits(out_local.numpy()), bits(out_full.numpy()[r0:r0 + rc]))
        db = g.sum_axis0(out_local).numpy()
        if backend == "nccl":  # the same column sum with its exchange inside the kernel: the NCCL path's bits, several in a row
            assert g.enable_peer_exchange(), gdev.plugin.last_error()
            for _ in range(5):
                assert np.array_equal(bits(g.sum_axis0(out_local).numpy()), bits(db))
            wide = Tensor.from_numpy(np.tile(out_local.numpy(), (1, 170)), gdev)  # 4080 columns: nearly the largest result the windows carry
            assert wide.shape[1] == 4080 and np.array_equal(bits(g.sum_axis0(wide).numpy()), bits(np.tile(db, 170)))
            g.disable_peer_exchange()
        parts = []
        for r in range(world):
            s, c = split_rows(rows, r, world)
            parts.append(out_full.numpy()[s:s + c].astype(np.float32))
        want_db = Tensor.from_numpy(
            np.stack([Tensor.from_numpy(p, dev).raw_sum_axis(0).numpy() for p in parts]), dev).raw_sum_axis(0).numpy()
        assert np.array_equal(bits(db), bits(want_db))
        assert np.allclose(db, out_full.numpy().astype(np.float64).sum(axis=0), rtol=0, atol=1e-5 * np.abs(out_full.numpy()).sum(axis=0).max())
    finally:
        dist.destroy_process_group()


def _layer_worker(rank: int, world: int, port: int):
    """Config 3 with its layers dealt to the ranks: the union of the ranks' updated parameters must be
    the single-device step's parameters, bit for bit (the placement it follows:
    crates/core/src/strategy.rs:269-326; the update: crates/python/python/pytorches/optim.py:13-16)."""
    sys.path.insert(0, ROOT)
    os.environ["PYTORCHES_CPU_THREADS"] = "2"
    from pytorches_b200.abi import Plugin
    from pytorches_b200.configs import config3_sharded, split_layers_of
    from pytorches_b200.core import Device

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        dev = Device(Plugin(ORACLE_SO), 0)
        layers, width, batch = 5, 96, 8  # uneven over 2 and 3 ranks
        _, _, mine = config3_sharded(dev, rank, world, layers, width, batch)()
        _, _, every = config3_sharded(dev, 0, 1, layers, width, batch)()
        own = split_layers_of(layers, rank, world)
        assert len(mine) == 2 * len(own)
        for k, l in enumerate(own):
            for j in range(2):  # weight, bias
                assert mine[2 * k + j].numpy().tobytes() == every[2 * l + j].numpy().tobytes(), f"layer {l} tensor {j}"
        counts = [None] * world
        dist.all_gather_object(counts, len(mine))
        assert sum(counts) == 2 * layers  # every parameter tensor has exactly one owner
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_layer_sharded_sgd_over_gloo(oracle, world):
    mp.spawn(_layer_worker, args=(world, _free_port()), nprocs=world, join=True)


@pytest.mark.parametrize("world,n", [(2, 200_001), (3, 70_000)])
def test_sharded_ops_over_gloo(oracle, world, n):
    mp.spawn(_worker, args=(world, _free_port(), n), nprocs=world, join=True)


@pytest.mark.gpu
@pytest.mark.parametrize("world,n", [(2, 200_001), (2, 1 << 22)])
def test_sharded_ops_over_nccl(oracle, b200, world, n):
    """The same checks with the B200 plugin on every rank and NCCL as the exchange (needs 2 GPUs)."""
    if b200.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), n, "nccl"), nprocs=world, join=True)


def test_split_rows_covers_everything():
    from pytorches_b200.shard import split_rows

    for n in (0, 1, 7, 8, 12, 1 << 28):
        for world in (1, 2, 3, 4, 8):
            spans = [split_rows(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1


def test_unsplit_order_rule(oracle, monkeypatch):
    """When may a sharded sum promise the bits of the unsplit sum? Pure host logic: every rank's shard must
    be a run of whole 65536-element blocks (the last one may end ragged), hold at least one, and the
    tensor must fit the window's block area; every rank must reach the same answer."""
    from pytorches_b200.core import Device
    from pytorches_b200.shard import ShardGroup

    def answers(n, world):
        out = []
        for rank in range(world):
            g = ShardGroup(Device(oracle, 0), rank, world)
            g._peer_reduce = object()  # as if the in-kernel exchange were on
            out.append(g.unsplit_order(n))
        assert len(set(out)) == 1
        return out[0]

    B = 65536
    for world in (1, 2, 4, 8):
        assert answers(1 << 28, world)               # the benchmark's tensor
        assert answers(B * world * 3, world)
        assert not answers(0, world)
        assert not answers((B << 14) + B, world)     # more blocks than the window holds
    assert answers(B * 3 + 5, 1)                     # one rank: any length
    assert not answers(B * 8 + 2 * 17, 2)            # rank 1 would start inside a block
    assert not answers(B, 2)                         # rank 1 would hold nothing
    assert not answers(B * 7, 2)                     # 3.5 blocks each
    monkeypatch.setenv("PYTORCHES_B200_UNSPLIT_ORDER", "0")
    assert not answers(1 << 28, 2)
    g = ShardGroup(Device(oracle, 0), 0, 2)          # without the in-kernel exchange there is no such promise
    monkeypatch.delenv("PYTORCHES_B200_UNSPLIT_ORDER")
    assert not g.unsplit_order(1 << 28)
