"""N-sharded Gemm on GPUs: every rank computes a block of output columns with the tile kernel, NCCL gathers the
blocks, the strided-copy kernel interleaves them.  Checked against the oracle's whole Gemm.  Runs with one rank on
any GPU box and with two ranks where two GPUs are visible."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
pytestmark = pytest.mark.gpu


def _case(dtype_name):
    import cases
    from espdl_b200 import abi
    if dtype_name == "int8":
        return cases.gemm_case(seed=21, dtype=abi.DTYPE_INT8, m=300, k=160, n_out=256, per_channel=True, e_out=-5)
    return cases.gemm_case(seed=22, dtype=abi.DTYPE_INT16, m=300, k=160, n_out=256, e_in=-14, e_w=(-15, -15), e_out=-12,
                           wide=True, bias_mag=1 << 20)


def _expected(case):
    import cases
    import checkers
    out = np.zeros_like(case["out"])
    assert checkers.oracle().oracle_conv2d(cases.conv_desc(dict(case, out=out))) == 0
    return out.reshape(case["in_w"], case["out_c"])


def _worker(rank, world, port, dtype_name, mode, ret):
    sys.path.insert(0, HERE)
    import conftest  # noqa: F401
    from espdl_b200 import abi, sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    abi.check(abi.load().espdl_b200_init(rank), "espdl_b200_init")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        c = _case(dtype_name)
        ew = c["ew"] if c["per_channel"] else c["filter_exponent"]
        gemm = sharding.NShardedGemm(c["w"].reshape(c["out_c"], c["in_c"]), c["b"], c["in_exponent"], ew,
                                     c["out_exponent"], activation=c["activation"], mode=mode)
        x = torch.from_numpy(c["x"].reshape(c["in_w"], c["in_c"])).cuda()
        out = gemm.forward(x)
        torch.cuda.synchronize()
        first = out.cpu().numpy().copy()
        out2 = gemm.forward(x)              # buffers are reused from the second call on
        torch.cuda.synchronize()
        assert np.array_equal(out2.cpu().numpy(), first)
        # consecutive calls on different inputs with no host synchronisation in between: each result is consumed on
        # the stream (a clone) while the next call's kernels - on this and on the other GPUs - are already enqueued
        xs = [x, torch.flip(x, dims=[0]), torch.roll(x, shifts=7, dims=0)]
        results = [gemm.forward(xi).clone() for xi in xs for _ in range(2)]
        torch.cuda.synchronize()
        first_rows = first
        for i, r in enumerate(results):
            want_rows = [first_rows, first_rows[::-1], np.roll(first_rows, 7, axis=0)][i // 2]
            assert np.array_equal(r.cpu().numpy(), want_rows), f"call {i} differs"
        ret.put((rank, first))
        gemm.close()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("dtype_name,mode", [("int8", "gather"), ("int16", "gather"), ("int8", "peer")])
@pytest.mark.parametrize("world", [1, 2])
def test_n_sharded_gemm_equals_whole_gemm(world, dtype_name, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, dtype_name, mode, ret)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(ret.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    sys.path.insert(0, HERE)
    want = _expected(_case(dtype_name))
    for r in range(world):
        np.testing.assert_array_equal(got[r], want)
