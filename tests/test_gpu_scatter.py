"""fl_fp8_linear_scatter: the product written by the epilogue into a column block of several
full-width matrices. On one GPU the destinations are two local matrices; with two or more GPUs a
second test maps a peer process's matrix through the IPC handle and checks the fused all-gather of
an output-channel split against the unsplit oracle."""
import os
import socket
import sys

import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def test_column_block_lands_in_every_destination(flint, oracle):
    F = flint
    rng = np.random.default_rng(71)
    m, n, k, ld, col0 = 300, 136, 192, 400, 64
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes, scales = oracle.quantize_fp8_rows(randn(rng, (n, k), 0.02))
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    res = oracle.narrow(randn(rng, (m, n)), True)
    bf = F.DType.BFLOAT16
    canvas = np.full((m, ld), 0x7FC0, np.uint16)  # NaN canvas: untouched columns must stay as they were
    d0, d1 = dev(F, canvas, bf), dev(F, canvas, bf)
    F.fp8_linear_scatter(dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT), [d0, d1], col0,
                         dev(F, bias, bf), dev(F, res, bf), F.ACT_GELU_TANH)
    got0, got1 = d0.numpy(), d1.numpy()
    F.synchronize()
    want = oracle.fp8_linear(x, codes, scales, bias, res, oracle.ACT_GELU_TANH)
    assert np.array_equal(got0, got1)
    check_parity(oracle, got0[:, col0:col0 + n], want, True, what="scatter block")
    mask = np.ones(ld, bool)
    mask[col0:col0 + n] = False
    assert np.all(got0[:, mask] == 0x7FC0), "columns outside the block were written"
    with pytest.raises(F.FlintError):
        F.fp8_linear_scatter(dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT), [d0], ld - 8)


def _worker(rank, world, port):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from libwaifu_b200 import flint as F
    from libwaifu_b200 import sharding
    from oracle import oracle as O
    from helpers import check_parity as check
    torch.cuda.set_device(rank)
    F.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(5)  # the same on every rank
        m, n, k = 520, 512, 256
        x = O.narrow(rng.standard_normal((m, k)).astype(np.float32), True)
        codes, scales = O.quantize_fp8_rows((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        a, b = sharding.column_shard(n, world, rank, 128)
        bf = F.DType.BFLOAT16
        # storage another process can map is a weight's own memory, 2 MiB or more: the (m, n) matrix
        # is the head of such a block
        big_rows = 2056
        own_block = F.Tensor.empty((big_rows, n), bf, hint=F.AllocHint.WEIGHT)
        own = own_block.view_as((m, n), (n, 1))
        handles = [None] * world
        dist.all_gather_object(handles, F.ipc_export(own_block))
        peers = [F.ipc_import(handles[r], (big_rows, n), bf) for r in range(world) if r != rank]
        dests = [own] + [p.view_as((m, n), (n, 1)) for p in peers]
        F.fp8_linear_scatter(F.Tensor.from_numpy(x, bf), F.Tensor.from_numpy(codes[a:b], F.DType.FP8E4M3),
                             F.Tensor.from_numpy(scales[a:b], F.DType.FLOAT), dests, a, None, None, F.ACT_GELU_TANH)
        flag = torch.zeros(1, device="cuda")
        dist.all_reduce(flag)  # every rank's pushes have landed once this has completed
        torch.cuda.synchronize()
        got = own.numpy()
        check(O, got, O.fp8_linear(x, codes, scales, None, None, O.ACT_GELU_TANH), True, what=f"rank {rank}")
        dist.barrier()
        del dests, peers
    finally:
        dist.destroy_process_group()


def test_fused_all_gather_across_gpus(flint, oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        mp.spawn(_worker, args=(2, port), nprocs=2, join=True)
    finally:
        os.environ.clear()
        os.environ.update(env)
