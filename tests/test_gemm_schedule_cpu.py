"""The tile kernel's schedule, checked without a GPU: fl_sm100_gemm_plan() gives the numbers a
launch would use, and the walk every role of a CTA makes over them (mirrored here from
gemm_sm100.cu's WorkWalk) must cover every K stage of every tile exactly once; a tile cut by the
stream-K part must have exactly two holders, neighbouring units, the head being the earlier unit's
last item and the tail the later unit's first, which is what the kernel's workspace slots and its
two-arrival counters rely on."""
import ctypes

import pytest

from libwaifu_b200 import flint as F

KINDS = {"half": 0, "bf16": 1, "e4m3": 2, "nvfp4": 3}


def plan(kind, m, n, k, sms, allow=1):
    out = (ctypes.c_int32 * 8)()
    F.check(F.lib().fl_sm100_gemm_plan(KINDS[kind], m, n, k, sms, allow, out))
    return dict(zip(("ctas", "block_n", "tiles", "num_kb", "units", "dp_rounds", "sk_tiles", "sk_first_tile"), out))


def walk(p, unit):
    """The items of one unit: (tile, kb0, kb1, partial, head)."""
    items = []
    for r in range(p["dp_rounds"]):
        tile = r * p["units"] + unit
        if tile >= p["tiles"]:
            break
        items.append((tile, 0, p["num_kb"], False, False))
    total = p["sk_tiles"] * p["num_kb"]
    pos, end = total * unit // p["units"], total * (unit + 1) // p["units"]
    while pos < end:
        t, kb0 = divmod(pos, p["num_kb"])
        length = min(end - pos, p["num_kb"] - kb0)
        items.append((p["sk_first_tile"] + t, kb0, kb0 + length, length != p["num_kb"], kb0 == 0))
        pos += length
    return items


SHAPES = [("e4m3", 4352, 12288, 3072), ("e4m3", 4352, 3072, 12288), ("e4m3", 4096, 3072, 3072), ("e4m3", 8704, 9216, 3072),
          ("e4m3", 8704, 3072, 3072), ("e4m3", 8704, 12288, 3072), ("e4m3", 8704, 3072, 12288), ("nvfp4", 4352, 9216, 3072),
          ("bf16", 4096, 12288, 3072), ("e4m3", 1024, 12288, 3072), ("e4m3", 520, 328, 1024), ("e4m3", 130, 264, 208),
          ("e4m3", 8192, 3072, 64), ("e4m3", 300, 200, 256), ("half", 513, 64, 64), ("e4m3", 19200, 256, 512),
          ("e4m3", 2, 18432, 3072), ("e4m3", 77 * 256, 256, 1024), ("e4m3", 149 * 128, 128, 2048)]


@pytest.mark.parametrize("sms", [148, 132, 16, 2])
@pytest.mark.parametrize("kind,m,n,k", SHAPES)
def test_every_stage_of_every_tile_is_computed_once(kind, m, n, k, sms):
    p = plan(kind, m, n, k, sms)
    assert p["units"] == min(p["tiles"], sms // p["ctas"])
    assert p["sk_tiles"] == 0 or p["sk_tiles"] >= p["units"]
    assert p["dp_rounds"] * p["units"] == p["sk_first_tile"] or p["sk_tiles"] == 0
    covered = {}
    holders = {}
    for u in range(p["units"]):
        items = walk(p, u)
        for index, (tile, kb0, kb1, partial, head) in enumerate(items):
            assert 0 <= tile < p["tiles"] and 0 <= kb0 < kb1 <= p["num_kb"]
            for kb in range(kb0, kb1):
                assert (tile, kb) not in covered, f"stage {kb} of tile {tile} computed twice"
                covered[(tile, kb)] = u
            if partial:
                # a part is the head (from stage 0) or the tail (to the last stage), never the middle
                assert (kb0 == 0) != (kb1 == p["num_kb"])
                assert head == (kb0 == 0)
                # the head is its unit's last item, the tail its unit's first item of the stream-K part
                if head:
                    assert index == len(items) - 1
                else:
                    assert index == min(p["dp_rounds"], len(items) - 1) or index == p["dp_rounds"]
                holders.setdefault(tile, []).append((u, head))
    assert len(covered) == p["tiles"] * p["num_kb"]
    for tile, parts in holders.items():
        assert len(parts) == 2, f"tile {tile} is cut into {len(parts)} parts"
        (u0, h0), (u1, h1) = sorted(parts)
        assert h0 and not h1 and u1 == u0 + 1, f"tile {tile}: head in unit {u0} ({h0}), tail in unit {u1} ({h1})"
    # workspace bounds the kernel indexes: two slots per unit, a counter set per stream-K tile
    assert p["sk_tiles"] <= 2 * p["units"]


def test_the_benchmark_shapes_use_the_stream_k_part_and_small_ones_do_not():
    up = plan("e4m3", 4352, 12288, 3072, 148)
    assert (up["ctas"], up["block_n"], up["tiles"], up["units"]) == (2, 256, 816, 74)
    assert (up["dp_rounds"], up["sk_tiles"], up["sk_first_tile"]) == (10, 76, 740)
    down = plan("e4m3", 4352, 3072, 12288, 148)
    assert (down["tiles"], down["dp_rounds"], down["sk_tiles"]) == (204, 1, 130)
    # without a workspace, or when the last round is nearly full, tiles stay whole
    assert plan("e4m3", 4352, 12288, 3072, 148, allow=0)["sk_tiles"] == 0
    assert plan("e4m3", 520, 328, 1024, 148)["sk_tiles"] == 0          # fewer tiles than units
    nearly_full = plan("e4m3", 256 * 73, 512, 1024, 148)               # 146 tiles on 74 units: 72 of 74 in the last round
    assert nearly_full["sk_tiles"] == 0 and nearly_full["dp_rounds"] == 2
    assert plan("e4m3", 8192, 3072, 64, 148)["sk_tiles"] == 0           # one K stage per tile: nothing to deal out
