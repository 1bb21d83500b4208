"""Host logic of the multi-GPU placement on CPU: row-shard arithmetic, the in-place gather of
row shards (world_size 2, gloo), the reference's --layer-map grammar, and the layer-split walk
with its hand-offs.  No GPU and no GEMV here: ranks fill their shards with known values."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import __graft_entry__ as graft
    graft.load_package()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _spawn(fn, world=2):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), fn, ret), nprocs=world, join=True)
    return dict(ret)


def test_shard_rows(pkg):
    from sycl_infer_b200.sharding import shard_rows
    assert shard_rows(5120, 0, 1) == (0, 5120)
    assert [shard_rows(17408, r, 8) for r in (0, 7)] == [(0, 2176), (15232, 17408)]
    assert shard_rows(1024, 3, 4) == (768, 1024)
    with pytest.raises(ValueError):
        shard_rows(1000, 0, 8)  # not a whole number of 16-row tiles per rank
    with pytest.raises(ValueError):
        shard_rows(1024, 4, 4)


def _gather_case(rank, world):
    from sycl_infer_b200.sharding import gather_rows, shard_rows
    out = {}
    for TB in (1, 3):
        n, col0, stride = 64, 32, 128
        full = torch.full((TB, stride), -1.0)
        r0, r1 = shard_rows(n, rank, world)
        for t in range(TB):
            full[t, col0 + r0:col0 + r1] = torch.arange(r0, r1, dtype=torch.float32) + 1000 * t
        gather_rows(full, n, col0, rank, world)
        out[TB] = full.numpy().copy()
    return out


def test_gather_rows_world2():
    res = _spawn(_gather_case, 2)
    for rank in (0, 1):
        for TB in (1, 3):
            got = res[rank][TB]
            for t in range(TB):
                assert np.array_equal(got[t, 32:96], np.arange(64, dtype=np.float32) + 1000 * t)
                assert np.all(got[t, :32] == -1) and np.all(got[t, 96:] == -1)


def test_layer_map_grammar(pkg):
    from sycl_infer_b200.sharding import even_layer_map, parse_layer_map, rank_of_layer
    r = parse_layer_map("0-31:gpu.0,32-63:gpu.1", 64)
    assert [(e.l0, e.l1, e.device) for e in r] == [(0, 32, "gpu.0"), (32, 64, "gpu.1")]
    assert parse_layer_map("0-3:gpu,4-7:cpu", 8)[1].device == "cpu"
    assert rank_of_layer(r, 40) == 1
    assert even_layer_map(64, 4) == "0-15:gpu.0,16-31:gpu.1,32-47:gpu.2,48-63:gpu.3"
    for bad, msg in (("0-31:gpu.0,33-63:gpu.1", "without gaps"), ("0-31:gpu.0", "layer count"),
                     ("0-31", "begin-end:device"), ("0-31:tpu", "gpu[.N] or cpu"), ("", "empty"),
                     ("5-2:gpu", "range")):
        with pytest.raises(ValueError, match=msg.replace("[", r"\[").replace("]", r"\]")):
            parse_layer_map(bad, 64)


def _split_case(rank, world):
    from sycl_infer_b200.sharding import even_layer_map, parse_layer_map, run_layer_split
    ranges = parse_layer_map(even_layer_map(6, world), 6)
    x = torch.zeros(2, 4)
    ran = []

    def run_layer(layer, x):
        ran.append(layer)
        x.mul_(2).add_(layer)  # order-sensitive: proves the layers ran in sequence across ranks

    run_layer_split(ranges, rank, x, run_layer)
    return ran, x.numpy().copy()


def test_layer_split_world2():
    res = _spawn(_split_case, 2)
    assert res[0][0] == [0, 1, 2] and res[1][0] == [3, 4, 5]
    v = 0.0
    for layer in range(6):
        v = 2 * v + layer
    assert np.all(res[1][1] == v)  # the last rank holds the result of all six layers


@pytest.mark.parametrize("world", [2, 4, 8])
def test_config1_layer_shards_at_every_bench_width(pkg, world):
    """Every projection of the benchmark layer splits into equal 16-row-aligned shards at 2, 4
    and 8 ranks, and the shards tile the rows exactly (what bench.py --gpus N relies on)."""
    from sycl_infer_b200.sharding import shard_rows
    for name, t, n, K in pkg.synth.dense_layer_shapes("Q4_K_M", hidden=5120, n_head=40, n_kv=8, head_dim=128, n_ff=17408):
        edges = [shard_rows(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert len({hi - lo for lo, hi in edges}) == 1 and (edges[0][1] - edges[0][0]) % 16 == 0


def test_gather_rows_world4():
    res = _spawn(_gather_case, world=4)
    for rank in range(4):
        for TB in (1, 3):
            got = res[rank][TB]
            for t in range(TB):
                assert np.array_equal(got[t, 32:96], np.arange(64, dtype=np.float32) + 1000 * t)
                assert np.all(got[t, :32] == -1) and np.all(got[t, 96:] == -1)
