"""The boundary's storage, transfers and elementwise operators on the card, through the C ABI:
stream-ordered storage (flint/cuda/cuda_tensor_data.cc:36-77), fl_transfer_async and its waits
(flint/capi.h:256-276), fl_copy / fl_cast / fl_fill / fl_add (flint/capi.h:246-249,279,483) against
numpy on the same bits, and the reporting path of a kernel whose bounded wait gave up."""
import ctypes
from ctypes import byref, c_int32, c_void_p

import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def host_pinned(F, arr, dtype):
    t = F.Tensor.empty(arr.shape, dtype, F.Device.CUDA_HOST)
    p = c_void_p()
    F.check(F.lib().fl_tensor_data_get_host_ptr(t._data, byref(p)))
    ctypes.memmove(p.value, np.ascontiguousarray(arr).ctypes.data, arr.nbytes)
    return t, p.value


def test_pool_storage_is_reused_without_growing_the_card(flint):
    """Create/destroy cycles of activation storage come out of the pool: after the first cycle the
    card's free memory does not move, and a block freed in stream order is handed out again."""
    import torch
    F = flint
    F.synchronize()
    t = F.Tensor.empty((1 << 20,), F.DType.FLOAT)
    del t
    F.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(50):
        t = F.Tensor.empty((1 << 20,), F.DType.FLOAT)
        F.fill(t, 1.0)
        del t
    F.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0


def test_only_a_weights_own_memory_can_be_exported(flint):
    F = flint
    small = F.Tensor.empty((1024,), F.DType.FLOAT, hint=F.AllocHint.WEIGHT)      # below 2 MiB: pooled
    pooled = F.Tensor.empty((1 << 20,), F.DType.FLOAT)                           # an activation: pooled
    own = F.Tensor.empty((1 << 20,), F.DType.FLOAT, hint=F.AllocHint.WEIGHT)     # 4 MiB weight: memory of its own
    for t in (small, pooled):
        with pytest.raises(F.FlintError) as e:
            F.ipc_export(t)
        assert e.value.code == F.FL_ERROR_INVALID_ARG
    assert len(F.ipc_export(own)) == 64


@pytest.mark.parametrize("shape", [(37,), (64, 520), (3, 5, 17)])
def test_cast_fill_add_copy_match_numpy(flint, oracle, shape):
    F, O = flint, oracle
    rng = np.random.default_rng(11)
    a32 = randn(rng, shape)
    b32 = randn(rng, shape)
    kinds = {F.DType.FLOAT16: False, F.DType.BFLOAT16: True}
    for dt, is_bf16 in kinds.items():
        a16, b16 = O.narrow(a32, is_bf16), O.narrow(b32, is_bf16)
        # float -> 16-bit rounds to nearest even, 16-bit -> float is exact
        got = F.cast(dev(F, a32, F.DType.FLOAT), dt).numpy()
        assert np.array_equal(got, a16)
        back = F.cast(dev(F, a16, dt), F.DType.FLOAT).numpy()
        assert np.array_equal(back, O.widen(a16, is_bf16))
        # the sum of two 16-bit values, one rounding
        want = O.narrow(O.widen(a16, is_bf16) + O.widen(b16, is_bf16), is_bf16)
        assert np.array_equal(F.add(dev(F, a16, dt), dev(F, b16, dt)).numpy(), want)
        t = F.Tensor.empty(shape, dt)
        F.fill(t, 0.3)
        assert np.array_equal(t.numpy(), O.narrow(np.full(shape, 0.3, np.float32), is_bf16))
    other = F.cast(dev(F, O.narrow(a32, False), F.DType.FLOAT16), F.DType.BFLOAT16).numpy()
    assert np.array_equal(other, O.narrow(O.widen(O.narrow(a32, False), False), True))
    assert np.array_equal(F.add(dev(F, a32, F.DType.FLOAT), dev(F, b32, F.DType.FLOAT)).numpy(), a32 + b32)
    c = F.Tensor.empty(shape, F.DType.FLOAT)
    F.copy(dev(F, a32, F.DType.FLOAT), c)
    assert np.array_equal(c.numpy(), a32)


def test_strided_and_broadcast_operands(flint, oracle):
    """A bias expanded over rows as a zero-stride view (what the Rust wrapper hands over,
    waifu/src/flint/functional.rs:80-108), and a transposed source for copy and cast."""
    F, O = flint, oracle
    rng = np.random.default_rng(12)
    a = O.narrow(randn(rng, (33, 72)), True)
    bias = O.narrow(randn(rng, (72,)), True)
    bf = F.DType.BFLOAT16
    got = F.add(dev(F, a, bf), dev(F, bias, bf)).numpy()
    assert np.array_equal(got, O.narrow(O.widen(a, True) + O.widen(bias, True)[None, :], True))
    src = dev(F, a, bf)
    transposed = src.view_as((72, 33), (1, 72))
    out = F.Tensor.empty((72, 33), bf)
    F.copy(transposed, out)
    assert np.array_equal(out.numpy(), a.T)
    assert np.array_equal(F.cast(transposed, F.DType.FLOAT).numpy(), O.widen(a, True).T)
    with pytest.raises(F.FlintError):
        F.cast(dev(F, np.zeros((4, 4), np.uint8), F.DType.UINT8), F.DType.FLOAT)
    with pytest.raises(F.FlintError):
        F.add(dev(F, a, bf), dev(F, a[:, :8].copy(), bf).view_as((33, 8), (8, 1)), F.Tensor.empty((33, 72), bf))


def test_asynchronous_upload_and_download_round_trip(flint):
    F = flint
    rng = np.random.default_rng(13)
    x = randn(rng, (257, 96))
    hx, _ = host_pinned(F, x, F.DType.FLOAT)
    d, pending = F.transfer_async(hx)
    pending.wait()       # the compute stream waits for the copy; the host does not
    doubled = F.add(d, d)
    hy, hy_ptr = host_pinned(F, np.zeros_like(x), F.DType.FLOAT)
    down = F.transfer_to_host_async(doubled, hy)
    down.wait_sync()     # now the host may read
    got = np.ctypeslib.as_array(ctypes.cast(hy_ptr, ctypes.POINTER(ctypes.c_float)), shape=x.shape)
    assert np.array_equal(got, x + x)
    # a transfer that nobody waits on may be destroyed, and its storage after it
    d2, pending2 = F.transfer_async(hx)
    del pending2, d2
    # wait_sync on an upload is the form for a host about to launch on another stream
    d3, pending3 = F.transfer_async(hx)
    pending3.wait_sync()
    assert np.array_equal(d3.numpy(), x)
    # pageable memory is refused rather than copied synchronously under an asynchronous name
    pageable = F.Tensor.from_numpy(x, F.DType.FLOAT, F.Device.CPU)
    with pytest.raises(F.FlintError) as e:
        F.transfer_async(pageable)
    assert "cuda-host to cuda" in e.value.message
    F.synchronize()


def test_a_wait_that_runs_out_is_reported_and_the_context_lives_on(flint, oracle):
    """The whole chain behind every bounded wait of the kernels: the wait gives up, the kernel
    writes its status and returns, the next synchronisation reports FL_ERROR_ABORTED with that
    status, and the call after it works. The kernel that gives up is a one-warp self-test waiting on
    a barrier nobody arrives on; the GEMM's own limit is not touched."""
    F, L = flint, flint.lib()
    F.synchronize()
    F.check(L.fl_sm100_selftest_wait_timeout(64))
    status = c_int32(0)
    assert L.fl_sm100_synchronize(byref(status)) == F.FL_ERROR_ABORTED
    assert status.value == 0x51
    assert b"gave up on a bounded wait" in L.fl_get_last_error_message()
    assert L.fl_sm100_synchronize(byref(status)) == F.FL_OK and status.value == 0
    # reported by the next operation too, when no synchronisation comes first
    a = dev(F, np.zeros((8, 32), np.uint16), F.DType.FLOAT16)
    w = dev(F, np.zeros((8, 32), np.uint8), F.DType.FP8E4M3)
    s = dev(F, np.ones(1, np.float32), F.DType.FLOAT)
    F.check(L.fl_sm100_selftest_wait_timeout(8))
    import torch
    torch.cuda.synchronize()
    with pytest.raises(F.FlintError) as e:
        F.fp8_matmul(a, w, s)
    assert e.value.code == F.FL_ERROR_ABORTED
    out = F.fp8_matmul(a, w, s).numpy()   # and the one after it runs
    assert not out.any()
    F.synchronize()


def test_the_static_arrays_status_word_is_reported_by_synchronize_and_transfer(flint, oracle):
    F, L = flint, flint.lib()
    rng = np.random.default_rng(14)
    x = oracle.narrow(randn(rng, (24, 64)), True)
    codes, scales = oracle.quantize_fp8_rows(randn(rng, (16, 64), 0.02))
    bf = F.DType.BFLOAT16
    xd, cd, sd = dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT)
    out = F.Tensor.empty((24, 16), bf)
    F.fp8_linear_static(xd, cd, sd, None, None, F.ACT_NONE, out)
    F.synchronize()                                   # nothing gave up
    F.check(L.fl_sm100_selftest_set_static_status(0x33))
    status = c_int32(0)
    assert L.fl_sm100_synchronize(byref(status)) == F.FL_ERROR_ABORTED and status.value == 0x33
    assert L.fl_sm100_synchronize(byref(status)) == F.FL_OK and status.value == 0
    F.check(L.fl_sm100_selftest_set_static_status(0x34))
    with pytest.raises(F.FlintError) as e:
        out.numpy()                                   # a transfer towards the host checks it too
    assert e.value.code == F.FL_ERROR_ABORTED and "fl_fp8_linear_static" in e.value.message
    got = out.numpy()                                 # cleared: the next one goes through
    check_parity(oracle, got, oracle.fp8_linear(x, codes, scales, None, None, 0), True, what="static 24x16x64")
    F.fp8_linear_static(xd, cd, sd, None, None, F.ACT_NONE, out)   # and the entry point itself still runs
    F.synchronize()


def test_a_second_device_in_one_process_is_refused(flint):
    F, L = flint, flint.lib()
    F.synchronize()
    import torch
    current = torch.cuda.current_device()
    assert L.fl_sm100_set_device(current) == F.FL_OK          # the same ordinal again is fine
    assert L.fl_sm100_set_device(current + 1) == F.FL_ERROR_INVALID_ARG
    assert b"one device per process" in L.fl_get_last_error_message()
