"""How the quantized-linear path is split over the GPUs of one box.

The reference runs on one GPU (device 0 is hard-wired, flint/cuda/cuda_operators.cc:91-96) and runs
the two classifier-free-guidance passes one after the other (waifu/src/qwen_image/pipeline.rs:
911-925). Two splits follow from the shape of the work:

* rows: images and guidance branches are independent, so the activation's rows are divided among
  the ranks, every rank keeps the whole weight, and nothing is exchanged (``row_shard``);
* columns: a large weight (rows, k) is divided by output channel, every rank multiplies the whole
  activation by its slice, and the slices of the result are all-gathered along the last dimension
  (``column_shard``, ``ColumnSplitLinear``). The all-gather is the one real exchange step.

One process per GPU; ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) is the plumbing.
The arithmetic of a rank is whatever ``linear`` callable it is given: the C-ABI ``fl_fp8_linear``
on a GPU, the CPU oracle in the tests.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple


def row_shard(m: int, world: int, rank: int, granule: int = 1) -> Tuple[int, int]:
    """[start, stop) of the rows rank `rank` owns: contiguous, sizes differing by at most one
    granule (a granule is the rows that must stay together, e.g. the tokens of one image)."""
    if m % granule != 0:
        raise ValueError(f"{m} rows are not whole granules of {granule}")
    units = m // granule
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * granule, stop * granule


def column_shard(n: int, world: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """[start, stop) of the output channels rank `rank` owns. Every slice is a multiple of
    `multiple` wide (8 is what the kernels read; 128 keeps attention heads whole)."""
    if n % multiple != 0:
        raise ValueError(f"{n} output channels are not a multiple of {multiple}")
    return row_shard(n, world, rank, granule=multiple)


def column_sizes(n: int, world: int, multiple: int = 8) -> List[int]:
    out = []
    for r in range(world):
        a, b = column_shard(n, world, r, multiple)
        out.append(b - a)
    return out


def all_gather_columns(dist, local, sizes: Sequence[int], out=None):
    """All-gathers (m, n_r) slices into (m, sum n_r), slice r at its column offset.

    With equal slices this is one ``all_gather_into_tensor`` into a (world, m, n_r) staging buffer
    followed by one strided copy into the row-major result (the layout the next GEMM's TMA reads);
    ragged slices are padded to the widest for the trip."""
    import torch
    m = local.shape[0]
    world = len(sizes)
    total = int(sum(sizes))
    if out is None:
        out = torch.empty((m, total), dtype=local.dtype, device=local.device)
    local = local.contiguous()
    if len(set(sizes)) == 1:
        stage = torch.empty((world * m, sizes[0]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(stage, local)  # rank r's slice lands in rows [r m, (r + 1) m)
        out.view(m, world, sizes[0]).copy_(stage.view(world, m, sizes[0]).permute(1, 0, 2))
    else:
        # Ragged slices: every rank pads its slice to the widest one so that the collective moves
        # equal pieces, and the padding is dropped on arrival.
        widest = max(sizes)
        padded = torch.zeros((m, widest), dtype=local.dtype, device=local.device)
        padded[:, :local.shape[1]].copy_(local)
        stage = torch.empty((world * m, widest), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(stage, padded)
        off = 0
        for r, s in enumerate(sizes):
            out[:, off:off + s].copy_(stage[r * m:(r + 1) * m, :s])
            off += s
    return out


class ColumnSplitLinear:
    """One linear layer split by output channel over the ranks of `dist`.

    `linear(x, weight_slice, scales_slice, bias_slice, residual_slice, act)` computes this rank's
    (m, n_r) slice; `forward` all-gathers the slices into the full (m, n)."""

    def __init__(self, dist, n: int, linear: Callable, multiple: int = 8):
        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.n = n
        self.sizes = column_sizes(n, self.world, multiple)
        self.start, self.stop = column_shard(n, self.world, self.rank, multiple)
        self.linear = linear

    def slice_of(self, full):
        """This rank's rows of a (n, ...) weight-side tensor (weight, per-channel scales, bias)."""
        return None if full is None else full[self.start:self.stop]

    def columns_of(self, full):
        """This rank's columns of an (m, n) activation-side tensor (a residual)."""
        return None if full is None else full[:, self.start:self.stop]

    def forward(self, x, weight_slice, scales_slice, bias_slice=None, residual_slice=None, act: int = 0, out=None):
        local = self.linear(x, weight_slice, scales_slice, bias_slice, residual_slice, act)
        return all_gather_columns(self.dist, local, self.sizes, out)


class NarrowGatherMlp:
    """An MLP split by output channel whose hidden activation crosses the links as e4m3 codes.

    The up projection's result H is only ever read by the down projection's activation quantiser,
    which turns a row of H into e4m3 codes and one scale, the row's largest magnitude over ALL its
    columns divided by 448. Gathering H in 16 bits and quantising afterwards moves twice the bytes
    it has to. Here every rank
      1. computes its column block of H and the largest magnitude of each row over that block
         (``up``: fl_fp8_linear_amax),
      2. takes the maximum of those over the ranks (one all-reduce of m floats),
      3. quantises its block with the whole row's scale and writes the codes into every rank's
         full-width matrix of codes (``scatter_codes``: fl_fp8_quantize_scatter over peer-mapped
         storage; the CPU tests all-gather instead),
      4. multiplies the gathered codes by its slice of the down weight (``down``:
         fl_fp8_linear_quantized, whose epilogue writes Y into every rank's matrix in the scatter
         form, or whose slices are all-gathered).
    The codes and scales equal what the unsplit chain's quantiser makes of the whole row, and a
    linear's output channels are independent, so the result equals the unsplit MLP's bit for bit.

    `ops` supplies the four callables; `dist` the collective for step 2."""

    def __init__(self, dist, n_up: int, n_down: int, multiple: int = 128):
        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.up_range = column_shard(n_up, self.world, self.rank, multiple)
        self.down_range = column_shard(n_down, self.world, self.rank, multiple)
        self.up_sizes = column_sizes(n_up, self.world, multiple)
        self.down_sizes = column_sizes(n_down, self.world, multiple)

    def step(self, x, up, scatter_codes, down):
        """`up(x) -> (h_block, row_amax tensor)`; `scatter_codes(h_block, row_amax, col0) -> (codes, scales)`
        (the full-width codes as this rank will read them, and the rows' scales);
        `down(codes, scales, col0) -> y`. Returns what `down` returns."""
        h_block, amax = up(x)
        self.dist.all_reduce(amax, op=self.dist.ReduceOp.MAX)
        codes, scales = scatter_codes(h_block, amax, self.up_range[0])
        return down(codes, scales, self.down_range[0])


def qkv_head_rows(heads: int, head_dim: int, world: int, rank: int) -> List[Tuple[int, int]]:
    """The rows of a fused (3 * heads * head_dim, k) QKV weight, laid out [q heads | k heads | v heads]
    (waifu/src/qwen_image/dit.rs:239-263), that rank `rank` owns when the projection is split on head
    boundaries: the same heads [h0, h1) of each of q, k and v, so that the rank can normalise, rotate
    and attend over its heads without any exchange. Three [start, stop) ranges."""
    h0, h1 = row_shard(heads, world, rank)
    return [(part * heads * head_dim + h0 * head_dim, part * heads * head_dim + h1 * head_dim) for part in range(3)]


class HeadSplitAttentionBlock:
    """QKV projection, attention and out projection of one stream, split over the ranks by head.

    Every rank projects the whole activation onto its heads of q, k and v (``qkv_head_rows``),
    normalises, rotates and attends over those heads alone, and holds a column block of the
    attention result (its heads' columns). The out projection reads whole rows, quantised per row:
    the block crosses the links as e4m3 codes exactly as the hidden activation of
    ``NarrowGatherMlp`` does (rows' maxima over the block, maximum over the ranks, codes written into
    every rank's full-width matrix), and every rank multiplies the gathered codes by its slice of the
    out projection's output channels. Heads, rows of a quantiser and output channels are all
    independent, so the result equals the unsplit chain bit for bit."""

    def __init__(self, dist, heads: int, head_dim: int, n_out: int, multiple: int = 128):
        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.heads = row_shard(heads, self.world, self.rank)
        self.qkv_rows = qkv_head_rows(heads, head_dim, self.world, self.rank)
        self.head_dim = head_dim
        self.col_range = (self.heads[0] * head_dim, self.heads[1] * head_dim)
        self.col_sizes = [(row_shard(heads, self.world, r)[1] - row_shard(heads, self.world, r)[0]) * head_dim
                          for r in range(self.world)]
        self.out_range = column_shard(n_out, self.world, self.rank, multiple)
        self.out_sizes = column_sizes(n_out, self.world, multiple)

    def step(self, x, qkv, attend, row_amax, scatter_codes, out_proj):
        """`qkv(x) -> this rank's (m, 3, heads_r, head_dim)`; `attend(qkv_r) -> (m, heads_r * head_dim)`;
        `row_amax(a_r) -> tensor of m maxima`; `scatter_codes(a_r, amax, col0) -> (codes, scales)`;
        `out_proj(codes, scales, col0) -> y`. Returns what `out_proj` returns."""
        a_block = attend(qkv(x))
        amax = row_amax(a_block)
        self.dist.all_reduce(amax, op=self.dist.ReduceOp.MAX)
        codes, scales = scatter_codes(a_block, amax, self.col_range[0])
        return out_proj(codes, scales, self.out_range[0])


def gather_rows(dist, local, sizes: Sequence[int]):
    """Concatenates row shards (used to hand a whole batch back to one caller)."""
    import torch
    widest = max(sizes)
    world = len(sizes)
    padded = torch.zeros((widest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[:local.shape[0]].copy_(local)
    stage = torch.empty((world * widest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(stage, padded)
    return torch.cat([stage[r * widest:r * widest + s] for r, s in enumerate(sizes)], dim=0)
