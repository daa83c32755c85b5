"""Multi-process path on CPU: two `gloo` ranks each run their shard of the batch through a golden model (with the
oracle standing in for the GPU forward) and gather the logits; the result must equal the single-process run."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
MODEL = os.path.join(HERE, "golden", "espdl", "c__linear_ishap_1_64_kshap_32_64_relu_s8.espdl")


def _forward(x):
    import graph_oracle
    from espdl_b200 import espdl_file
    m = espdl_file.read(MODEL)
    name_in, name_out = m["inputs"][0]["name"], m["outputs"][0]["name"]
    return graph_oracle.run_graph(m, {name_in: x})[name_out]


def _worker(rank, world, port, total, ret):
    sys.path.insert(0, HERE)
    import conftest  # noqa: F401  (registers the package under its import name)
    from espdl_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = np.random.default_rng(5).integers(-128, 128, size=(total, 64), dtype=np.int8)
        b, e = sharding.shard_range(total, rank, world)
        local = torch.from_numpy(_forward(x[b:e]).reshape(e - b, -1).copy())
        full = sharding.gather_logits(local, total)
        if rank == 0:
            ret.put(full.numpy())
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("total", [8, 7])  # equal shards, ragged shards
def test_two_ranks_equal_one(total):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, total, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = np.random.default_rng(5).integers(-128, 128, size=(total, 64), dtype=np.int8)
    np.testing.assert_array_equal(got, _forward(x).reshape(total, -1))


def test_shard_range_covers_everything_once():
    from espdl_b200 import sharding
    for total in (0, 1, 7, 8, 1000, 1025):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _columns_worker(rank, world, port, ret):
    sys.path.insert(0, HERE)
    import conftest  # noqa: F401
    from espdl_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = np.random.default_rng(9).integers(-128, 128, size=(5, 12), dtype=np.int8)
        n_loc = 12 // world
        local = torch.from_numpy(full[:, rank * n_loc:(rank + 1) * n_loc].copy())
        got = sharding.gather_columns(local)
        ret.put((rank, got.numpy()))
    finally:
        dist.destroy_process_group()


def test_column_blocks_gather_into_the_whole_matrix():
    """N-sharded Gemm exchange: each rank owns a block of output columns; every rank ends with [M][N]."""
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_columns_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(ret.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = np.random.default_rng(9).integers(-128, 128, size=(5, 12), dtype=np.int8)
    for r in range(2):
        np.testing.assert_array_equal(got[r], full)
