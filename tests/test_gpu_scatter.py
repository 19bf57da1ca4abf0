"""fl_fp8_linear_scatter: the product written by the epilogue into a column block of several
full-width matrices. On one GPU the destinations are two local matrices; with two or more GPUs a
second test maps a peer process's matrix through the IPC handle and checks the fused all-gather of
an output-channel split against the unsplit oracle."""
import ctypes
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


def _narrow_worker(rank, world, port):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from libwaifu_b200 import flint as F
    from libwaifu_b200 import sharding
    from oracle import oracle as O
    torch.cuda.set_device(rank)
    F.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(6)  # the same on every rank
        m, d, n_up = 520, 256, 512
        x = O.narrow(rng.standard_normal((m, d)).astype(np.float32), True)
        up_c, up_s = O.quantize_fp8_rows((rng.standard_normal((n_up, d)) * 0.02).astype(np.float32))
        dn_c, dn_s = O.quantize_fp8_rows((rng.standard_normal((d, n_up)) * 0.02).astype(np.float32))
        bf, f8, fl = F.DType.BFLOAT16, F.DType.FP8E4M3, F.DType.FLOAT
        dev = lambda a, dt: F.Tensor.from_numpy(a, dt, F.Device.CUDA)
        mlp = sharding.NarrowGatherMlp(dist, n_up, d, multiple=128)
        (ua, ub), (da, db) = mlp.up_range, mlp.down_range
        # the full-width matrix of codes every rank writes its block into: storage of its own
        # allocation (2 MiB or more), the only kind another process can map
        big_rows = 4104
        codes_block = F.Tensor.empty((big_rows, n_up), f8, hint=F.AllocHint.WEIGHT)
        y_block = F.Tensor.empty((big_rows, d), bf, hint=F.AllocHint.WEIGHT)
        handles = [None] * world
        dist.all_gather_object(handles, (F.ipc_export(codes_block), F.ipc_export(y_block)))
        peers = [(F.ipc_import(handles[r][0], (big_rows, n_up), f8), F.ipc_import(handles[r][1], (big_rows, d), bf))
                 for r in range(world) if r != rank]
        codes_own = codes_block.view_as((m, n_up), (n_up, 1))
        y_own = y_block.view_as((m, d), (d, 1))
        codes_dests = [codes_own] + [p[0].view_as((m, n_up), (n_up, 1)) for p in peers]
        y_dests = [y_own] + [p[1].view_as((m, d), (d, 1)) for p in peers]
        xd = dev(x, bf)
        w_up, s_up = dev(up_c[ua:ub], f8), dev(up_s[ua:ub], fl)
        w_dn, s_dn = dev(dn_c[da:db], f8), dev(dn_s[da:db], fl)
        x_cols = dev(np.ascontiguousarray(x[:, da:db]), bf)
        amax_t = torch.zeros(m, device="cuda", dtype=torch.float32)
        amax = F.Tensor.from_device_ptr(amax_t.data_ptr(), (m,), fl, keepalive=amax_t)
        scales = F.Tensor.empty((m,), fl)

        def all_gather_handles(mine):
            every = [None] * world
            dist.all_gather_object(every, mine)
            return every

        group = F.PeerGroup(rank, world, m, all_gather_handles)

        class InKernelMax:
            """What NarrowGatherMlp asks of `dist`: the maximum over the ranks, here by the library's own
            exchange kernel on the stream (no library collective between the GEMMs)."""
            ReduceOp = dist.ReduceOp
            get_world_size, get_rank = staticmethod(dist.get_world_size), staticmethod(dist.get_rank)

            @staticmethod
            def all_reduce(t, op=None):
                assert t is amax_t and op == dist.ReduceOp.MAX
                group.exchange(amax)

        mlp.dist = InKernelMax

        def up_op(_):
            return F.fp8_linear_amax(xd, w_up, s_up, amax, None, None, F.ACT_GELU_TANH), amax_t

        def scatter_op(h_block, amax_tensor, col0):
            F.fp8_quantize_scatter(h_block, amax, codes_dests, col0, scales)
            group.exchange()  # every rank's block of codes has landed once this has completed
            return codes_own, scales

        def down_op(codes, row_scales, col0):
            F.fp8_linear_quantized_scatter(codes, row_scales, w_dn, s_dn, y_dests, col0, None, x_cols, F.ACT_NONE)
            group.exchange()
            return y_own

        for _ in range(3):  # the buffers and mailboxes are reused step after step
            mlp.step(xd, up_op, scatter_op, down_op)
        F.synchronize()
        got_codes = codes_own.numpy()
        h_ref = O.fp8_linear(x, up_c, up_s, None, None, O.ACT_GELU_TANH)
        want_codes, want_scales = O.quantize_fp8_act(h_ref, True)
        # H is the GPU's and may differ from the oracle's in a last place here and there, which moves
        # a code or, where it is the row's largest value, a scale: nearly all agree
        same_scales = float(np.mean(scales.numpy().view(np.uint32) == want_scales.view(np.uint32)))
        same = float(np.mean(got_codes == want_codes))
        assert same_scales >= 0.9 and same >= 0.9, f"rank {rank}: {same_scales:.3f} of the scales, {same:.4f} of the codes equal the oracle's"
        y_ref = O.fp8_linear(h_ref, dn_c, dn_s, None, x, O.ACT_NONE)
        got_y = y_own.numpy()
        check_parity_local(O, got_y, y_ref, f"rank {rank}: the whole MLP, codes gathered and Y scattered")
        # the gathered codes and scales are the same bytes on every rank
        digest = torch.tensor([float(got_codes.astype(np.uint64).sum()), float(scales.numpy().astype(np.float64).sum()),
                               float(got_y.astype(np.uint64).sum())],
                              device="cuda", dtype=torch.float64)
        both = [torch.zeros_like(digest) for _ in range(world)]
        dist.all_gather(both, digest)
        assert all(torch.equal(b, both[0]) for b in both), "the ranks hold different codes, scales or results"
        dist.barrier()
        del codes_dests, y_dests, peers, group
    finally:
        dist.destroy_process_group()


def check_parity_local(O, got16, want16, what):
    from helpers import check_parity as check
    check(O, got16, want16, True, what=what)


def test_narrow_gather_across_gpus(flint, oracle):
    """The hidden activation of a column-split MLP gathered as e4m3 codes over peer-mapped storage
    (fl_fp8_linear_amax, a maximum over the ranks, fl_fp8_quantize_scatter), on two GPUs."""
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
        mp.spawn(_narrow_worker, args=(2, port), nprocs=2, join=True)
    finally:
        os.environ.clear()
        os.environ.update(env)


def test_row_maxima_and_quantise_scatter_on_one_gpu(flint, oracle):
    """fl_fp8_linear_amax leaves the rows' largest rounded magnitudes; fl_fp8_quantize_scatter with
    those maxima writes, block by block, exactly the codes and scales fl_quantize_fp8_activation makes
    of the whole matrix."""
    F = flint
    rng = np.random.default_rng(72)
    m, n, k = 300, 384, 192
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes, scales = oracle.quantize_fp8_rows(randn(rng, (n, k), 0.02))
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    bf, f8, fl = F.DType.BFLOAT16, F.DType.FP8E4M3, F.DType.FLOAT
    amax = F.Tensor.empty((m,), fl)
    h = F.fp8_linear_amax(dev(F, x, bf), dev(F, codes, f8), dev(F, scales, fl), amax, dev(F, bias, bf), None, F.ACT_GELU_TANH)
    h_np = h.numpy()
    assert np.array_equal(amax.numpy(), oracle.row_amax(h_np, True))
    check_parity(oracle, h_np, oracle.fp8_linear(x, codes, scales, bias, None, oracle.ACT_GELU_TANH), True, what="with row maxima")
    # two column blocks of h scattered into two full-width matrices of codes
    d0 = dev(F, np.full((m, n), 0x7F, np.uint8), f8)
    d1 = dev(F, np.full((m, n), 0x7F, np.uint8), f8)
    row_scales = F.Tensor.empty((m,), fl)
    for (a, b) in [(0, 256), (256, 384)]:
        block = dev(F, np.ascontiguousarray(h_np[:, a:b]), bf)
        F.fp8_quantize_scatter(block, amax, [d0, d1], a, row_scales)
    want_codes, want_scales = oracle.quantize_fp8_act(h_np, True)
    assert np.array_equal(d0.numpy(), want_codes) and np.array_equal(d1.numpy(), want_codes)
    assert np.array_equal(row_scales.numpy().view(np.uint32), want_scales.view(np.uint32))
    with pytest.raises(F.FlintError):
        F.fp8_quantize_scatter(dev(F, np.ascontiguousarray(h_np[:, :256]), bf), amax, [d0], 136)   # does not fit / not a multiple of 16


def test_peer_exchange_with_a_peer_written_by_the_host(flint, oracle):
    """One GPU, two mailboxes: this rank's and a stand-in for a peer's. The peer's flag and payload
    are put into this rank's mailbox by a copy before the kernel runs (no second kernel waits on this
    one), so the kernel finds its peer arrived, and leaves the larger of the two maxima per row."""
    F = flint
    rows, world, width = 300, 2, F.PEER_HEADER + 320
    rng = np.random.default_rng(8)
    mine = np.abs(rng.standard_normal(rows)).astype(np.float32)
    theirs = np.abs(rng.standard_normal(rows)).astype(np.float32)
    box0 = np.zeros((world, width), np.int32)
    box0[1, 0] = 7                                   # the peer's flag, already at this epoch
    box0[1, F.PEER_HEADER:F.PEER_HEADER + rows] = theirs.view(np.int32)
    own = F.Tensor.from_numpy(box0, F.DType.INT32)
    peer = F.Tensor.from_numpy(np.zeros((world, width), np.int32), F.DType.INT32)
    amax = F.Tensor.from_numpy(mine, F.DType.FLOAT)
    arr = (ctypes.c_void_p * 2)(own.raw(), peer.raw())
    F.check(F.lib().fl_sm100_peer_exchange(arr, 2, 0, 7, amax.raw(), 0))
    F.synchronize()
    assert np.array_equal(amax.numpy(), np.maximum(mine, theirs))
    got_peer = peer.numpy()
    assert got_peer[0, 0] == 7 and np.array_equal(got_peer[0, F.PEER_HEADER:F.PEER_HEADER + rows].view(np.float32), mine)
    assert own.numpy()[0, 0] == 7
    # a later epoch passes too when the flag is already ahead of it; an earlier argument is refused
    F.check(F.lib().fl_sm100_peer_exchange(arr, 1, 0, 8, None, 0))
    F.synchronize()
    for bad in [(arr, 0, 0, 1), (arr, 2, 2, 1), (arr, 2, 0, 0)]:
        assert F.lib().fl_sm100_peer_exchange(bad[0], bad[1], bad[2], bad[3], None, 0) == F.FL_ERROR_INVALID_ARG


def test_peer_exchange_gives_up_on_a_peer_that_never_arrives(flint):
    """The wait is bounded: a peer whose flag nothing sets makes the kernel record its status and
    return; the next synchronisation reports it and the library carries on."""
    F, L = flint, flint.lib()
    world, width = 2, F.PEER_HEADER + 16
    own = F.Tensor.from_numpy(np.zeros((world, width), np.int32), F.DType.INT32)
    peer = F.Tensor.from_numpy(np.zeros((world, width), np.int32), F.DType.INT32)
    keep = np.arange(16, dtype=np.float32)
    amax = F.Tensor.from_numpy(keep, F.DType.FLOAT)
    arr = (ctypes.c_void_p * 2)(own.raw(), peer.raw())
    F.synchronize()
    F.check(L.fl_sm100_peer_exchange(arr, 2, 0, 1, amax.raw(), 64))
    status = ctypes.c_int32(0)
    assert L.fl_sm100_synchronize(ctypes.byref(status)) == F.FL_ERROR_ABORTED and status.value == 0x61
    assert L.fl_sm100_synchronize(ctypes.byref(status)) == F.FL_OK and status.value == 0
    assert np.array_equal(amax.numpy(), keep)


def test_row_maxima_of_a_column_block(flint, oracle):
    """fl_fp8_row_amax over a column block of a wider matrix (this rank's heads of an attention
    result) equals the oracle's maxima of the same block, for both 16-bit types."""
    F = flint
    rng = np.random.default_rng(73)
    for is_bf16, dt in ((True, F.DType.BFLOAT16), (False, F.DType.FLOAT16)):
        full = oracle.narrow(randn(rng, (70, 384), 3.0), is_bf16)
        d = dev(F, full, dt)
        for (a, b) in [(0, 384), (128, 256), (250, 381)]:   # the last neither aligned nor a multiple of 8
            block = d.view_as((70, b - a), (384, 1), a)
            got = F.fp8_row_amax(block).numpy()
            assert np.array_equal(got, oracle.row_amax(np.ascontiguousarray(full[:, a:b]), is_bf16)), (is_bf16, a, b)


def test_quantized_product_lands_in_every_destination(flint, oracle):
    """fl_fp8_linear_quantized_scatter on one GPU: codes and row scales in, the product (bias,
    residual, one rounding) in a column block of two full-width matrices, the rest of them untouched;
    the same bits as fl_fp8_linear_quantized gives on its own."""
    F = flint
    rng = np.random.default_rng(74)
    m, n, k, ld, col0 = 300, 136, 192, 400, 64
    x = oracle.narrow(randn(rng, (m, k)), True)
    a_codes, a_scales = oracle.quantize_fp8_act(x, True)
    codes, scales = oracle.quantize_fp8_rows(randn(rng, (n, k), 0.02))
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    res = oracle.narrow(randn(rng, (m, n)), True)
    bf, f8, fl = F.DType.BFLOAT16, F.DType.FP8E4M3, F.DType.FLOAT
    fill = np.full((m, ld), 0x7FC0, np.uint16)
    d0, d1 = dev(F, fill, bf), dev(F, fill, bf)
    ops = (dev(F, a_codes, f8), dev(F, a_scales, fl), dev(F, codes, f8), dev(F, scales, fl))
    F.fp8_linear_quantized_scatter(*ops, [d0, d1], col0, dev(F, bias, bf), dev(F, res, bf), F.ACT_GELU_TANH)
    alone = F.Tensor.empty((m, n), bf)
    F.fp8_linear_quantized(*ops, dev(F, bias, bf), dev(F, res, bf), F.ACT_GELU_TANH, alone)
    F.synchronize()
    want = oracle.fp8_linear_quantized(a_codes, a_scales, codes, scales, bias, res, oracle.ACT_GELU_TANH)
    for d in (d0, d1):
        got = d.numpy()
        assert np.array_equal(got[:, col0:col0 + n], alone.numpy())
        check_parity(oracle, got[:, col0:col0 + n], want, True, what="quantized scatter")
        assert (got[:, :col0] == 0x7FC0).all() and (got[:, col0 + n:] == 0x7FC0).all()
    with pytest.raises(F.FlintError):
        F.fp8_linear_quantized_scatter(*ops, [d0], ld - n + 8, None, None, F.ACT_NONE)   # does not fit
