"""The multi-GPU splits of the path, checked on CPU with two gloo ranks: each rank's arithmetic is
the CPU oracle, so what is under test is the host-side sharding (ranges, gathers, layouts) that the
GPU ranks use unchanged. Rows and output channels are independent in a quantized linear (the
activation is quantised per row, the weight per channel), so the sharded results must equal the
unsharded ones bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _as_t(a16):
    # gloo carries no 16-bit types: one 16-bit pattern per int32 for the trip
    return torch.from_numpy(np.ascontiguousarray(a16).astype(np.int32))


def _as_np(t):
    return np.ascontiguousarray(t.numpy()).astype(np.uint16)


def _worker(rank, world, port, ragged):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from libwaifu_b200 import sharding
    from oracle import oracle as O
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(99)  # the same on every rank
        m, k, n_up = 96, 128, (264 if ragged else 256)
        x = O.narrow(rng.standard_normal((m, k)).astype(np.float32), True)
        up_c, up_s = O.quantize_fp8_rows((rng.standard_normal((n_up, k)) * 0.02).astype(np.float32))
        dn_c, dn_s = O.quantize_fp8_rows((rng.standard_normal((k, n_up)) * 0.02).astype(np.float32))
        bias = O.narrow((rng.standard_normal(n_up) * 0.01).astype(np.float32), True)
        h_ref = O.fp8_linear(x, up_c, up_s, bias, None, O.ACT_GELU_TANH)
        y_ref = O.fp8_linear(h_ref, dn_c, dn_s, None, x, O.ACT_NONE)

        # ---- rows: no exchange until the results are collected
        sizes = [b - a for a, b in (sharding.row_shard(m, world, r, granule=16) for r in range(world))]
        a, b = sharding.row_shard(m, world, rank, granule=16)
        h_rows = O.fp8_linear(x[a:b], up_c, up_s, bias, None, O.ACT_GELU_TANH)
        y_rows = O.fp8_linear(h_rows, dn_c, dn_s, None, x[a:b], O.ACT_NONE)
        y_all = _as_np(sharding.gather_rows(dist, _as_t(y_rows), sizes))
        assert np.array_equal(y_all, y_ref), "row-sharded MLP differs from the unsharded one"

        # ---- output channels: all-gather after each linear
        def linear(xt, w, s, bt, rt, act):
            out = O.fp8_linear(_as_np(xt), w, s, None if bt is None else _as_np(bt), None if rt is None else _as_np(rt), act)
            return _as_t(out)

        up = sharding.ColumnSplitLinear(dist, n_up, linear)
        assert sum(up.sizes) == n_up and all(s % 8 == 0 for s in up.sizes)
        h = up.forward(_as_t(x), up.slice_of(up_c), up.slice_of(up_s), up.slice_of(_as_t(bias)), None, O.ACT_GELU_TANH)
        assert np.array_equal(_as_np(h), h_ref), "column-split up projection differs"
        down = sharding.ColumnSplitLinear(dist, k, linear)
        xt = _as_t(x)
        y = down.forward(h, down.slice_of(dn_c), down.slice_of(dn_s), None, down.columns_of(xt).contiguous(), O.ACT_NONE)
        assert np.array_equal(_as_np(y), y_ref), "column-split down projection differs"

        # ---- output channels with the hidden activation gathered as e4m3 codes
        mlp = sharding.NarrowGatherMlp(dist, n_up, k, multiple=8)
        assert (mlp.up_range, mlp.down_range) == ((up.start, up.stop), (down.start, down.stop))

        def up_op(x16):
            a0, b0 = mlp.up_range
            h_block = O.fp8_linear(x16, up_c[a0:b0], up_s[a0:b0], bias[a0:b0], None, O.ACT_GELU_TANH)
            return h_block, torch.from_numpy(O.row_amax(h_block, True).copy())

        def scatter_op(h_block, amax_t, col0):
            codes_block, scales = O.quantize_fp8_act_amax(h_block, amax_t.numpy(), True)
            gathered = sharding.all_gather_columns(dist, torch.from_numpy(codes_block.astype(np.int32)), mlp.up_sizes)
            return gathered.numpy().astype(np.uint8), scales

        def down_op(codes, scales, col0):
            a0, b0 = mlp.down_range
            y_block = O.fp8_linear_quantized(codes, scales, dn_c[a0:b0], dn_s[a0:b0], None, x[:, a0:b0], O.ACT_NONE)
            return _as_np(sharding.all_gather_columns(dist, _as_t(y_block), mlp.down_sizes))

        y_narrow = mlp.step(x, up_op, scatter_op, down_op)
        assert np.array_equal(y_narrow, y_ref), "the MLP with e4m3-gathered hidden activation differs from the unsharded one"

        # ---- QKV split on head boundaries, attention on a rank's own heads, the out projection on
        # ---- the attention result gathered as e4m3 codes
        heads, hd, tokens, batch = 4, 32, 24, 2
        hidden, rows = heads * hd, batch * tokens
        xa = O.narrow(rng.standard_normal((rows, hidden)).astype(np.float32), True)
        qkv_c, qkv_s = O.quantize_fp8_rows((rng.standard_normal((3 * hidden, hidden)) * 0.05).astype(np.float32))
        out_c, out_s = O.quantize_fp8_rows((rng.standard_normal((hidden, hidden)) * 0.05).astype(np.float32))
        ang = np.outer(np.arange(tokens), 1.0 / (10000.0 ** (np.arange(hd // 2) / (hd // 2)))).astype(np.float32)
        cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)

        def attend(qkv16, n_heads):
            """(rows, 3 * n_heads * hd) -> (rows, n_heads * hd): norm and rotation, then attention per image."""
            r = O.qk_norm_rope(qkv16, cos, sin, n_heads, 1e-6, True)
            five = r.reshape(batch, tokens, 3, n_heads, hd)
            q, kk, v = (np.ascontiguousarray(five[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
            a = O.narrow(O.attention(q, kk, v, False, True).astype(np.float32), True)       # (batch, heads, tokens, hd)
            return np.ascontiguousarray(a.transpose(0, 2, 1, 3)).reshape(rows, n_heads * hd)

        a_ref = attend(O.fp8_linear(xa, qkv_c, qkv_s, None, None, O.ACT_NONE), heads)
        y_attn_ref = O.fp8_linear(a_ref, out_c, out_s, None, xa, O.ACT_NONE)
        blk = sharding.HeadSplitAttentionBlock(dist, heads, hd, hidden, multiple=8)
        mine = np.concatenate([np.arange(a0, b0) for a0, b0 in blk.qkv_rows])
        assert len(mine) == 3 * (blk.heads[1] - blk.heads[0]) * hd

        def qkv_op(x16):
            return O.fp8_linear(x16, qkv_c[mine], qkv_s[mine], None, None, O.ACT_NONE)

        def attend_op(qkv_block):
            return attend(qkv_block, blk.heads[1] - blk.heads[0])

        def amax_op(a_block):
            return torch.from_numpy(O.row_amax(a_block, True).copy())

        def scatter_attn(a_block, amax_t, col0):
            assert col0 == blk.col_range[0]
            codes_block, scales = O.quantize_fp8_act_amax(a_block, amax_t.numpy(), True)
            gathered = sharding.all_gather_columns(dist, torch.from_numpy(codes_block.astype(np.int32)), blk.col_sizes)
            return gathered.numpy().astype(np.uint8), scales

        def out_op(codes, scales, col0):
            a0, b0 = blk.out_range
            y_block = O.fp8_linear_quantized(codes, scales, out_c[a0:b0], out_s[a0:b0], None, xa[:, a0:b0], O.ACT_NONE)
            return _as_np(sharding.all_gather_columns(dist, _as_t(y_block), blk.out_sizes))

        y_attn = blk.step(xa, qkv_op, attend_op, amax_op, scatter_attn, out_op)
        assert np.array_equal(y_attn, y_attn_ref), "the head-split attention block differs from the unsplit one"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ragged", [False, True])
def test_two_ranks_match_one(ragged):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), ragged), nprocs=2, join=True)


def test_shard_ranges_cover_and_align():
    from libwaifu_b200 import sharding
    for m, world, g in [(4352, 8, 1), (4352 * 2, 8, 4352), (16, 3, 1), (9216, 8, 128), (12288, 7, 8)]:
        spans = [sharding.row_shard(m, world, r, g) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == m
        for (a0, b0), (a1, b1) in zip(spans, spans[1:]):
            assert b0 == a1
        assert all((b - a) % g == 0 for a, b in spans)
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= g
    with pytest.raises(ValueError):
        sharding.column_shard(100, 4, 0, multiple=8)
    # a fused QKV weight split on head boundaries: every rank the same heads of q, k and v, all rows taken once
    heads, hd = 24, 128
    seen = np.zeros(3 * heads * hd, np.int32)
    for r in range(8):
        spans = sharding.qkv_head_rows(heads, hd, 8, r)
        assert len(spans) == 3 and len({b - a for a, b in spans}) == 1 and all(a % hd == 0 and b % hd == 0 for a, b in spans)
        assert spans[1][0] - spans[0][0] == heads * hd and spans[2][0] - spans[1][0] == heads * hd
        for a, b in spans:
            seen[a:b] += 1
    assert (seen == 1).all()
